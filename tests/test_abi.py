"""CPU checks of the drop-in boundary: the shared library loads, exports every symbol the
header declares, rejects bad arguments before touching CUDA, and the capture modules keep
the reference's candidate-module contract.  No GPU work happens here."""

import ctypes
import json
import os
import pathlib
import re

import pytest

ROOT = pathlib.Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def lib():
    from mosaicist_b200 import build

    build.build()
    from mosaicist_b200 import _lib

    return _lib.load()


def _declared():
    text = "".join(p.read_text() for p in sorted((ROOT / "include").glob("*.h")))
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(msc_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(lib):
    from mosaicist_b200 import _lib

    names = _declared()
    assert len(names) >= 11
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/ but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert sorted(_lib.SIGNATURES) == names
    assert lib.msc_version() >= 1
    assert lib.msc_ptx_path().decode().endswith("libmosaicist_sm100a.ptx")
    assert pathlib.Path(lib.msc_ptx_path().decode()).exists()


def test_bad_arguments_are_rejected_with_a_message(lib):
    from mosaicist_b200 import _lib

    cfg = _lib.GemmCfg()
    one = ctypes.c_void_p(16)  # non-null, aligned; never dereferenced on these paths
    rc = lib.msc_grouped_gemm_nvfp4(None, one, one, one, None, None, one, 1, 128, 128, 64, cfg, None)
    assert rc == _lib.ERR_BAD_ARG and b"NULL" in lib.msc_last_error()
    rc = lib.msc_grouped_gemm_nvfp4(one, one, one, one, None, None, one, 1, 100, 128, 64, cfg, None)
    assert rc == _lib.ERR_BAD_ARG and b"multiple of 128" in lib.msc_last_error()
    rc = lib.msc_grouped_gemm_nvfp4(one, one, one, one, None, None, one, 1, 128, 128, 48, cfg, None)
    assert rc == _lib.ERR_BAD_ARG and b"k=48" in lib.msc_last_error()
    cfg.tile_n = 64
    rc = lib.msc_grouped_gemm_nvfp4(one, one, one, one, None, None, one, 1, 128, 128, 64, cfg, None)
    assert rc == _lib.ERR_UNSUPPORTED
    cfg.tile_n = 256
    rc = lib.msc_grouped_gemm_nvfp4(one, one, one, one, None, None, one, 1, 128, 384, 64, cfg, None)
    assert rc == _lib.ERR_BAD_ARG and b"tile_n" in lib.msc_last_error()
    rc = lib.msc_grouped_gemm_nvfp4_ragged(one, one, one, one, None, None, None, None, one, 1, 128,
                                           128, 64, None, None)
    assert rc == _lib.ERR_BAD_ARG and b"group_offsets" in lib.msc_last_error()
    rc = lib.msc_grouped_gemm_mxfp8_ragged(one, one, one, one, None, one, one, None, one, 1, 128,
                                           128, 96, None, None)
    assert rc == _lib.ERR_BAD_ARG
    rc = lib.msc_nvfp4_quantize(one, 0, one, None, one, one, 0, 1, 128, 100, None)
    assert rc == _lib.ERR_BAD_ARG and b"multiple of 64" in lib.msc_last_error()
    rc = lib.msc_sf_swizzle(one, one, 1, 128, 6, None)
    assert rc == _lib.ERR_BAD_ARG
    with pytest.raises(_lib.MscError) as e:
        _lib.check(rc)
    assert e.value.code == _lib.ERR_BAD_ARG


def test_candidate_module_contract(monkeypatch):
    import importlib

    m = importlib.import_module("mosaicist_b200.candidates.cand_cuda_gemm")
    assert callable(m.build) and callable(m.reference)
    assert all(isinstance(v, list) and v for v in m.KNOBS.values())
    assert {k: v[0] for k, v in m.KNOBS.items()} == m.DEFAULTS     # first value is the default
    assert set(m.STRUCTURAL) <= set(m.KNOBS)
    from mosaicist_b200.candidates._common import from_env

    monkeypatch.setenv("MOSAICIST_KNOBS", json.dumps({"tile_n": 256}))
    assert from_env(m.DEFAULTS)["tile_n"] == 256 and from_env(m.DEFAULTS)["stages"] == 0
    spec = json.loads((ROOT / "mosaicist_b200/candidates/spec_nvfp4_gemm.json").read_text())
    assert spec["dims"] == {"l": m.L, "m": m.M, "n": m.N, "k": m.K}
    assert spec["out_dtype"] == "bfloat16"


def test_moe_candidate_module_contract():
    import importlib

    m = importlib.import_module("mosaicist_b200.candidates.cand_cuda_moe")
    assert callable(m.build) and callable(m.reference)
    assert {k: v[0] for k, v in m.KNOBS.items()} == m.DEFAULTS and set(m.STRUCTURAL) <= set(m.KNOBS)
    spec = json.loads((ROOT / "mosaicist_b200/candidates/spec_nvfp4_moe.json").read_text())
    assert spec["dims"] == {"l": m.L, "m": m.M, "k": m.K, "n": m.N}


def test_candidate_module_against_reference_harness(monkeypatch):
    """When the reference checkout is present, its own loader and knob space accept the
    module unchanged."""
    from oracle.stage_reference import staged_path

    ref = staged_path()
    if ref is None:
        pytest.skip("the reference's package is neither staged (oracle/stage_reference.py) nor in MOSAICIST_REFERENCE")
    monkeypatch.syspath_prepend(str(ref))
    from mosaicist.capture import load_build
    from mosaicist.converge.knobs import KnobSpace
    import mosaicist_b200.candidates.cand_cuda_gemm as m

    assert load_build("mosaicist_b200.candidates.cand_cuda_gemm") is m.build
    assert KnobSpace.from_module(m).default() == m.DEFAULTS


def test_byte_decoders_match_ml_dtypes():
    import ml_dtypes
    import numpy as np

    from mosaicist_b200 import formats as F
    from oracle import nvfp4 as O

    allb = np.arange(256, dtype=np.uint8)
    assert np.array_equal(F.E4M3_LUT, allb.view(ml_dtypes.float8_e4m3fn).astype(np.float64), equal_nan=True)
    assert np.array_equal(F.E2M1_LUT, np.arange(16, dtype=np.uint8).view(ml_dtypes.float4_e2m1fn).astype(np.float64))
    rng = np.random.default_rng(3)
    q, sf = O.exact_operands(rng, 1, 200, 128)
    got = F.dequant_nvfp4(O.pack_e2m1(q[0]), O.e4m3_bytes(O.to_mma_scale_layout(sf[0])))
    want = q[0].astype(np.float64) * np.repeat(sf[0].astype(np.float64), 16, axis=-1)
    assert np.array_equal(got, want)


def test_profile_stage_summary_table():
    """The profiling stage's CSV folding: per kernel launches, average duration, DRAM GB/s."""
    from mosaicist_b200.profile_stage import METRICS, summarise

    head = '"ID","Process ID","Process Name","Host Name","Kernel Name","Context","Stream","Block Size","Grid Size","Device","CC","Section Name","Metric Name","Metric Unit","Metric Value"'
    rows = ["==PROF== Connected to process 1", head]
    vals = {0: [10000, 4_000_000, 1_000_000, 50.0, 30.0, 153, 15.0, 70_000_000],
            1: [30000, 8_000_000, 2_000_000, 60.0, 40.0, 153, 17.0, 90_000_000],
            2: [5000, 1_000_000, 0, 10.0, 0.0, 32, 80.0, 0]}
    names = {0: "gemm_pair_kernel<0, 5, 0, 0>(CUtensorMap)", 1: "gemm_pair_kernel<0, 5, 0, 0>(CUtensorMap)",
             2: "moe_plan_kernel(const int *)"}
    units = ["ns", "byte", "byte", "%", "%", "register/thread", "%", "byte"]
    for i, v in vals.items():
        for m, u, x in zip(METRICS, units, v):
            rows.append(f'"{i}","1","python","host","{names[i]}","1","7","(320, 1, 1)","(148, 1, 1)","0","10.0","Command line profiler metrics","{m}","{u}","{x}"')
    for i in (0, 1):
        rows.append(f'"{i}","1","python","host","{names[i]}","1","7","(320, 1, 1)","(148, 1, 1)","0","10.0","Command line profiler metrics","smsp__average_warps_issue_stalled_barrier_per_issue_active.ratio","","2.5"')
    table = summarise("\n".join(rows)).splitlines()
    assert table[2].startswith("| gemm_pair_kernel<0, 5, 0, 0> | 2 | 20.0 | 6.00 | 1.50 | 375 | 55.0 | 35.0 | 153 | 16.0 | 80.0 |")
    assert table[3].startswith("| moe_plan_kernel | 1 | 5.0 | 1.00 | 0.00 | 200 |")
    from mosaicist_b200.profile_stage import kernel_rows

    rows_ = kernel_rows("\n".join(rows))
    assert rows_[0]["top_stalls"][0] == {"reason": "barrier", "warps_per_issue_active": 2.5}


def test_expert_parallel_entry_points_reject_bad_arguments(lib):
    """Argument checks of the peer-memory exchange run before any CUDA call."""
    from mosaicist_b200 import _lib

    one = ctypes.c_void_p(256)
    two = (ctypes.c_void_p * 2)(256, 256)
    rc = lib.msc_ep_offsets(one, 3, 0, 32, 1024, one, one, one, one, None, 0, 0, None)
    assert rc == _lib.ERR_BAD_ARG and b"do not split" in lib.msc_last_error()
    rc = lib.msc_ep_offsets(one, 2, 2, 32, 1024, one, one, one, one, None, 0, 0, None)
    assert rc == _lib.ERR_BAD_ARG and b"rank=2" in lib.msc_last_error()
    rc = lib.msc_ep_offsets(one, 2, 0, 32, 1000, one, one, one, one, None, 0, 0, None)
    assert rc == _lib.ERR_BAD_ARG and b"rows_cap" in lib.msc_last_error()
    rc = lib.msc_ep_offsets(one, 17, 0, 34, 1024, one, one, one, one, None, 0, 0, None)
    assert rc == _lib.ERR_UNSUPPORTED and b"world=17" in lib.msc_last_error()
    rc = lib.msc_ep_dispatch_quantize(one, one, one, one, one, one, 8, 100, 2, 32, 2, two, two, two, None, None, 0,
                                      1024, one, None)
    assert rc == _lib.ERR_BAD_ARG and b"hidden=100" in lib.msc_last_error()
    rc = lib.msc_ep_dispatch_quantize(one, one, one, one, one, one, 1 << 24, 256, 8, 32, 2, two, two, two, None,
                                      None, 0, 1024, one, None)
    assert rc == _lib.ERR_UNSUPPORTED and b"26 bits" in lib.msc_last_error()
    rc = lib.msc_ep_dispatch_quantize(one, one, one, one, one, one, 8, 256, 2, 32, 2, two, two, two, None, two, 0,
                                      1024, one, None)
    assert rc == _lib.ERR_BAD_ARG and b"row_next needs row_dest" in lib.msc_last_error()
    rc = lib.msc_ep_presum_push(one, one, one, two, 17, 64, 128, 256, None)
    assert rc == _lib.ERR_BAD_ARG and b"dest_count=17" in lib.msc_last_error()
    rc = lib.msc_ep_combine(None, one, one, one, 8, 256, 2, 32, 2, 1024, None)
    assert rc == _lib.ERR_BAD_ARG and b"NULL" in lib.msc_last_error()
    rc = lib.msc_ep_sum_pairs(one, None, one, 8, 100, 2, None)
    assert rc == _lib.ERR_BAD_ARG and b"hidden=100" in lib.msc_last_error()
    cfg = _lib.GemmCfg()
    rc = lib.msc_grouped_gemm_nvfp4_scatter_ragged(one, one, one, one, None, one, one, None, one, two, 2, 64, 4, 512,
                                                   384, 256, cfg, None)
    assert rc == _lib.ERR_BAD_ARG and b"n=384" in lib.msc_last_error()
    rc = lib.msc_grouped_gemm_nvfp4_scatter_ragged(one, one, one, one, None, one, one, None, one, two, 17, 64, 4, 512,
                                                   256, 256, cfg, None)
    assert rc == _lib.ERR_UNSUPPORTED and b"dest_count=17" in lib.msc_last_error()
    rc = lib.msc_ep_offsets(one, 2, 0, 32, 1024, one, one, one, one, one, 9, 1, None)
    assert rc == _lib.ERR_BAD_ARG and b"slot=9" in lib.msc_last_error()
    rc = lib.msc_ep_signal(two, 2, 0, 4, 1, None, None, 0, None)
    assert rc == _lib.ERR_BAD_ARG and b"slot=4" in lib.msc_last_error()
    rc = lib.msc_ep_signal(two, 2, 0, 1, 1, one, None, 32, None)
    assert rc == _lib.ERR_BAD_ARG and b"counts need" in lib.msc_last_error()
    rc = lib.msc_ep_wait(None, 2, 0, 1, None)
    assert rc == _lib.ERR_BAD_ARG
    rc = lib.msc_peer_alloc(0, ctypes.byref(ctypes.c_void_p()), ctypes.create_string_buffer(64))
    assert rc == _lib.ERR_BAD_ARG


def test_torch_custom_op_is_registered_and_shape_propagates():
    """torch.ops.mosaicist_sm100a.grouped_gemm_nvfp4 exists after import and FakeTensor tracing
    sees its output shape / dtype without a GPU."""
    import torch
    from torch._subclasses.fake_tensor import FakeTensorMode

    import mosaicist_b200.torch_ops  # noqa: F401

    with FakeTensorMode():
        u8 = dict(dtype=torch.uint8, device="cuda")
        out = torch.ops.mosaicist_sm100a.grouped_gemm_nvfp4(
            torch.empty((8, 512, 1024), **u8), torch.empty((8, 4, 32, 32, 16), **u8),
            torch.empty((8, 2048, 1024), **u8), torch.empty((8, 16, 32, 32, 16), **u8), None, None)
        assert tuple(out.shape) == (8, 512, 2048) and out.dtype == torch.bfloat16
        x = torch.empty((8, 512, 2048), dtype=torch.bfloat16, device="cuda")
        gs = torch.empty((8,), dtype=torch.float32, device="cuda")
        q, sf = torch.ops.mosaicist_sm100a.quantize_nvfp4(x, gs, None)
        assert tuple(q.shape) == (8, 512, 1024) and tuple(sf.shape) == (8, 4, 32, 32, 16)
        q, sf = torch.ops.mosaicist_sm100a.silu_mul_quantize_nvfp4(x, gs, None)
        assert tuple(q.shape) == (8, 512, 512) and tuple(sf.shape) == (8, 4, 16, 32, 16)
        i32 = dict(dtype=torch.int32, device="cuda")
        y = torch.ops.mosaicist_sm100a.grouped_gemm_nvfp4_ragged(
            torch.empty((1024, 1024), **u8), torch.empty((8, 32, 32, 16), **u8), torch.empty((4, 512, 1024), **u8),
            torch.empty((4, 4, 32, 32, 16), **u8), torch.empty((4,), **i32), torch.empty((4,), **i32), None, None)
        assert tuple(y.shape) == (1024, 512) and y.dtype == torch.bfloat16
        gs = torch.ops.mosaicist_sm100a.global_scale_for(x)
        assert tuple(gs.shape) == (8,) and gs.dtype == torch.float32
        q, sf = torch.ops.mosaicist_sm100a.quantize_mxfp8(torch.empty((300, 512), dtype=torch.bfloat16, device="cuda"))
        assert tuple(q.shape) == (300, 512) and tuple(sf.shape) == (3, 4, 32, 16) and q.dtype == torch.uint8
        y = torch.ops.mosaicist_sm100a.grouped_gemm_mxfp8_ragged(
            torch.empty((1024, 1024), **u8), torch.empty((8, 8, 32, 16), **u8), torch.empty((4, 512, 1024), **u8),
            torch.empty((4, 4, 8, 32, 16), **u8), torch.empty((4,), **i32), torch.empty((4,), **i32), None, None)
        assert tuple(y.shape) == (1024, 512) and y.dtype == torch.bfloat16
        h = dict(dtype=torch.float16, device="cuda")
        c = torch.ops.mosaicist_sm100a.gemm_f16(torch.empty((256, 128), **h), torch.empty((128, 384), **h))
        assert tuple(c.shape) == (256, 384) and c.dtype == torch.float16
        y = torch.ops.mosaicist_sm100a.grouped_gemm_bf16_int4_ragged(
            torch.empty((768, 512), dtype=torch.bfloat16, device="cuda"), torch.empty((3, 256, 256), **u8),
            torch.empty((3, 256, 4), dtype=torch.bfloat16, device="cuda"), torch.empty((3,), **i32),
            torch.empty((3,), **i32), None, 128)
        assert tuple(y.shape) == (768, 256) and y.dtype == torch.bfloat16
        f32 = dict(dtype=torch.float32, device="cuda")
        y = torch.ops.mosaicist_sm100a.moe_masked(
            torch.empty((2, 256, 512), dtype=torch.bfloat16, device="cuda"), torch.empty((2, 512, 256), **u8),
            torch.empty((2, 4, 8, 32, 16), **u8), torch.empty((2,), **f32), torch.empty((2,), **f32),
            torch.empty((2, 512, 128), **u8), torch.empty((2, 4, 4, 32, 16), **u8), torch.empty((2,), **f32),
            torch.empty((2,), **f32), torch.empty((2,), **i32), torch.empty((2,), **f32), torch.empty((2,), **f32))
        assert tuple(y.shape) == (2, 256, 512) and y.dtype == torch.bfloat16


def test_dropped_ptx_is_reduced_to_the_running_instantiation(lib, tmp_path, monkeypatch):
    """The capture module leaves a PTX holding only the kernel instantiation that runs (the
    fingerprinter picks the entry with the most instructions)."""
    import re

    from mosaicist_b200.candidates import _common

    toy = (".version 8.8\n.target sm_100a\n.extern .shared .b8 s[];\n"
           ".visible .entry kA_ILi1E(\n .param .u64 p\n)\n{\n { nested } \n ret;\n}\n"
           ".visible .entry kB_ILi2E(\n .param .u64 p\n)\n.maxntid 320\n{\n ret;\n}\n")
    red = _common.only_entry(toy, "kB_ILi2E")
    assert "kB_ILi2E" in red and "kA_ILi1E" not in red and red.startswith(".version 8.8") and ".maxntid 320" in red
    assert _common.only_entry(toy, "missing") == toy
    monkeypatch.setenv("MOSAIC_GPU_DUMP_TO", str(tmp_path))
    _common.drop_artifacts("pair", "gemm_pair_kernelILi0ELi5ELb0ELb0ELb0E")
    text = next(tmp_path.glob("*.ptx")).read_text()
    entries = re.findall(r"^\.visible \.entry (\S+)\(", text, re.M)
    assert len(entries) == 1 and "gemm_pair_kernelILi0ELi5ELb0ELb0ELb0E" in entries[0]
    assert list(tmp_path.glob("ptxas*"))


def test_bench_reference_arm_runs_on_the_cpu_and_prints_the_contract_line():
    """`bench.py --impl reference` needs no GPU: one JSON line with the same metric, unit and
    workload as the GPU arm, the CPU baseline describing itself, and zero copied bytes."""
    import subprocess
    import sys

    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1",
                          "--warmup", "0"], capture_output=True, text=True, check=True, cwd=ROOT).stdout
    line = json.loads(out.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] == "nvfp4_grouped_gemm_tflops" and line["unit"] == "TFLOP/s"
    assert line["n_gpus"] == 1 and line["steps"] == 1 and line["higher_is_better"] is True
    assert "l=8 m=512 n=2048 k=2048" in line["config"]["workload"]
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["cpu_baseline"]["value"] == line["value"] > 0
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0


@pytest.mark.parametrize("kernel,entry", [("pair", "gemm_pair_kernelILi0ELi5ELb0ELb0ELb0E"),
                                          ("single", "gemm_blockscaled_kernelILi0ELi128ELi5E"),
                                          ("dense", "gemm_dense_f16_kernelILi6ELb0ELb0E")])
def test_reference_fingerprinter_accepts_the_dropped_ptx(kernel, entry, tmp_path, monkeypatch, lib):
    """What a capture module leaves in the dump directory goes through the reference's own PTX
    parser and fingerprinter (src/mosaicist/ptx/parse.py, features.py:151): it parses, its largest
    entry is the instantiation that was asked for, and the fingerprint sees tensor-core and TMA
    instructions."""
    from oracle.stage_reference import staged_path

    ref = staged_path()
    if ref is None:
        pytest.skip("the reference's package is neither staged (oracle/stage_reference.py) nor in MOSAICIST_REFERENCE")
    monkeypatch.syspath_prepend(str(ref))
    monkeypatch.setenv("MOSAIC_GPU_DUMP_TO", str(tmp_path))
    from mosaicist.ptx.features import fingerprint
    from mosaicist.ptx.parse import parse
    from mosaicist_b200.candidates._common import drop_artifacts

    drop_artifacts(kernel, entry)
    files = list(tmp_path.glob("*.ptx"))
    assert len(files) == 1
    text = files[0].read_text()
    mod = parse(text)
    assert entry in mod.entry(None).name and mod.target == "sm_100a"
    fp = fingerprint(text, ptxas_log=(tmp_path / "ptxas_mosaicist_sm100a.log").read_text())
    ops = " ".join(i.opcode for i in mod.entry(None).instrs)
    assert "tcgen05.mma" in ops and "cp.async.bulk.tensor" in ops
    assert fp is not None
