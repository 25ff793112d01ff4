// Expert-parallel token exchange over peer memory: every rank owns a contiguous block of the
// experts and a slice of the tokens, and the GPUs of one box see each other's receive buffers
// (CUDA IPC mappings over NVLink).  Instead of sorting rows by destination and calling a
// library all-to-all, the dispatch kernel quantises a token block once and stores the packed
// row and its routing weight straight into the owning rank's GEMM operand buffers, at the row
// the exchanged counts assign to it (the scale bytes go into a row-major buffer, 32-byte
// pieces over NVLink instead of scattered words, and the owner tiles them locally with
// msc_sf_swizzle); the combine kernel reads each
// token's expert outputs from the owners' result buffers and sums them.  The only collective
// left is the all-gather of the per-expert counts, plus two stream-ordered barriers the host
// places between the phases (pushes visible before the GEMMs, results complete before the
// pull).  No kernel here waits on another GPU.
//
// The reference has no multi-GPU code; the partitioning is the one its benchmark
// configuration names (expert-parallel across the GPUs of one box, dispatch and combine).
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "../../include/mosaicist_sm100a.h"
#include "host_common.h"
#include "ptx.cuh"
#include "quantize_common.cuh"

namespace msc {

constexpr int kMaxPeers = 16;
constexpr int kMaxSumTopk = 64;   // pairs of one token the final sum stages
constexpr uint32_t kStatusEpOverflow = 0x00E00000u;   // a destination row beyond rows_cap

// ---- signalling between ranks ----------------------------------------------------------------
// Each rank owns a small table of flags, 16 per slot, one per peer, that only the peers write
// (monotonically increasing epochs) and only the owner reads.  A signal is a system-scope
// release store into every peer's table after a system fence; it is launched after the kernels
// whose peer-memory writes it announces, so those writes have completed.  A wait spins, with a
// time limit, on the owner's own memory; nothing here blocks on another GPU's progress without
// that limit, and a wait that gives up raises a status bit and returns.
constexpr uint32_t kStatusEpWaitTimeout = 0x00D00000u;
constexpr int kFlagSlots = 4;   // a flag table is kFlagSlots x kMaxPeers ints
constexpr long long kEpWaitBudgetNs = 1000000000LL;   // one second

__device__ __forceinline__ void flag_store_release_sys(int* addr, int value) {
  asm volatile("st.release.sys.global.b32 [%0], %1;" ::"l"(addr), "r"(value) : "memory");
}
__device__ __forceinline__ int flag_load_acquire_sys(const int* addr) {
  int v;
  asm volatile("ld.acquire.sys.global.b32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Lanes below `world` each wait for one peer's flag of `slot` to reach `epoch`; true if all did.
__device__ __forceinline__ bool wait_for_peers(const int* flags, int world, int slot, int epoch,
                                               uint32_t* status) {
  bool ok = true;
  if ((int)threadIdx.x < world) {
    const int* f = flags + slot * kMaxPeers + threadIdx.x;
    const unsigned long long t0 = global_timer_ns();
    while (flag_load_acquire_sys(f) < epoch) {
      if ((long long)(global_timer_ns() - t0) > kEpWaitBudgetNs) {
        atomicOr(status, kStatusEpWaitTimeout);
        ok = false;
        break;
      }
      __nanosleep(200);
    }
  }
  return ok;
}

struct EpSignalParams {
  int* flags[kMaxPeers];        // every rank's flag table
  int* counts_all[kMaxPeers];   // every rank's (world, experts_total) table, or null entries
  const int* counts;            // this rank's (experts_total) counts, or null
  int world, rank, slot, epoch, experts_total;
};

// Optionally copies this rank's per-expert counts into row `rank` of every peer's table, then
// raises this rank's flag of `slot` on every peer.
__global__ void __launch_bounds__(256) ep_signal_kernel(const EpSignalParams p) {
  if (p.counts) {
    for (int i = threadIdx.x; i < p.world * p.experts_total; i += blockDim.x) {
      const int peer = i / p.experts_total, e = i - peer * p.experts_total;
      p.counts_all[peer][(size_t)p.rank * p.experts_total + e] = __ldg(p.counts + e);
    }
  }
  __threadfence_system();
  __syncthreads();
  if ((int)threadIdx.x < p.world)
    flag_store_release_sys(p.flags[threadIdx.x] + p.slot * kMaxPeers + p.rank, p.epoch);
}

__global__ void __launch_bounds__(32)
ep_wait_kernel(const int* flags, int world, int slot, int epoch, uint32_t* status) {
  wait_for_peers(flags, world, slot, epoch, status);
}

// ---- offsets ---------------------------------------------------------------------------------
// counts_all[s][e]: pairs rank s routes to global expert e.  One block computes, for every
// expert, the first row this rank's pairs take in the owner's buffers (the owner's 128-aligned
// group offset plus the pairs of lower ranks), and this rank's own group table.
__global__ void __launch_bounds__(256)
ep_offsets_kernel(const int* counts_all, int world, int rank, int experts_total,
                  int experts_local, int rows_cap, int* __restrict__ send_base,
                  int* __restrict__ group_rows, int* __restrict__ group_offsets,
                  int* __restrict__ total_rows, uint32_t* __restrict__ status,
                  const int* wait_flags, int wait_slot, int wait_epoch) {
  extern __shared__ int aligned_total[];   // experts_total entries
  if (wait_flags) {   // the counts arrive from the peers: wait for all of them to be published
    wait_for_peers(wait_flags, world, wait_slot, wait_epoch, status);
    __syncthreads();
  }
  for (int e = threadIdx.x; e < experts_total; e += blockDim.x) {
    int total = 0;
    for (int s = 0; s < world; ++s) total += __ldcg(counts_all + (size_t)s * experts_total + e);
    aligned_total[e] = (total + 127) & ~127;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < experts_total; e += blockDim.x) {
    const int owner = e / experts_local;
    int off = 0;
    for (int j = owner * experts_local; j < e; ++j) off += aligned_total[j];
    int before = 0, total = 0;
    for (int s = 0; s < world; ++s) {
      const int c = __ldcg(counts_all + (size_t)s * experts_total + e);
      if (s < rank) before += c;
      total += c;
    }
    send_base[e] = off + before;
    if (owner == rank) {
      // the table this rank's GEMMs walk never reaches beyond its buffers: a group that starts
      // at or after rows_cap gets no rows, one that straddles it is cut (its senders drop the
      // pairs that do not fit and the overflow bit below says so)
      const int el = e - owner * experts_local;
      group_rows[el] = off >= rows_cap ? 0 : min(total, rows_cap - off);
      group_offsets[el] = min(off, rows_cap);
      if (el == experts_local - 1) *total_rows = min(off + aligned_total[e], rows_cap);
    }
    if (e == (owner + 1) * experts_local - 1 && off + aligned_total[e] > rows_cap)
      atomicOr(status, kStatusEpOverflow);
  }
}

// ---- dispatch --------------------------------------------------------------------------------
struct EpDispatchParams {
  const __nv_bfloat16* tokens;   // (tokens, hidden)
  const int* ids;                // (tokens, topk) global expert ids
  const float* weights;          // (tokens, topk)
  const int* rank_in_group;      // (tokens, topk) position among this rank's pairs of the expert
  const int* send_base;          // (experts_total)
  const float* gs;               // (experts_total) input global scale of every expert
  int* pair_row;                 // (tokens, topk) out: row in the owner's buffers
  uint32_t* status;
  uint8_t* q[kMaxPeers];         // per rank: (rows_cap, hidden/2)
  uint8_t* sf[kMaxPeers];        // per rank: row-major (rows_cap, hidden/16)
  float* row_weight[kMaxPeers];  // per rank: (rows_cap)
  int* row_dest[kMaxPeers];      // per rank: (rows_cap) where the row's result goes, or all null
  int* row_next[kMaxPeers];      // per rank: (rows_cap) next row of the same token there, or all null
  int entries, hidden, topk, experts_total, experts_local, rows_cap, rank;
};

// One thread per (token, 16-value block), as in the single-GPU dispatch: the block is loaded
// once, quantised once per distinct global scale, and stored into every owner's buffers.
__global__ void __launch_bounds__(256) ep_dispatch_kernel(const EpDispatchParams p) {
  const int kblocks = p.hidden >> 4;
  const long long unit = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long token = unit / kblocks;
  const int kb = (int)(unit - token * kblocks);
  const bool live = token * p.topk < p.entries;
  float v[16];
  if (live) load16_bf16(p.tokens + (size_t)token * p.hidden + kb * 16, v);
  uint2 q8 = make_uint2(0u, 0u);
  uint32_t sfb = 0;
  float have_gs = -1.0f;
  for (int k = 0; k < p.topk; ++k) {
    const long long entry = token * p.topk + k;
    int e = -1;
    if (live) e = __ldg(p.ids + entry);
    bool valid = e >= 0 && e < p.experts_total;
    int dest = 0, owner = 0;
    if (valid) {
      owner = e / p.experts_local;
      dest = __ldg(p.send_base + e) + __ldg(p.rank_in_group + entry);
      if (dest < 0 || dest >= p.rows_cap) {   // never store outside the owner's buffers
        valid = false;
        if (kb == 0) {
          atomicOr(p.status, kStatusEpOverflow);
          p.pair_row[entry] = -1;   // the combine skips it
        }
      }
    }
    if (valid) {
      const float gs = __ldg(p.gs + e);
      if (gs != have_gs) {
        quantize_16(v, gs, q8, sfb);
        have_gs = gs;
      }
      *reinterpret_cast<uint2*>(p.q[owner] + (size_t)dest * (p.hidden >> 1) + kb * 8) = q8;
      if (kb == 0) {
        p.row_weight[owner][dest] = __ldg(p.weights + entry);
        if (p.row_dest[owner]) p.row_dest[owner][dest] = (p.rank << 26) | (int)entry;
        p.pair_row[entry] = dest;
      }
    }
    const uint32_t word = gather_scale_word(sfb);
    if (valid && (kb & 3) == 0)
      *reinterpret_cast<uint32_t*>(p.sf[owner] + (size_t)dest * kblocks + kb) = word;
  }
  // no fence here: the stores are complete when the grid is, and what announces them to the
  // other ranks (a signal kernel or a collective) is launched after this grid in the stream
}

// The same dispatch with the rows leaving as bulk copies: one block per token quantises the
// row into shared memory (3.5 KB of values + 448 scale bytes at hidden 7168) and one thread
// sends it to each of the token's experts as two untiled bulk copies, so NVLink sees a few
// large writes per row instead of hundreds of 8-byte stores.  The row is re-quantised only when
// an expert's global scale differs from the one in shared memory.  Needs hidden % 256 == 0
// (the scale row must be a multiple of 16 bytes).
__global__ void __launch_bounds__(256) ep_dispatch_bulk_kernel(const EpDispatchParams p) {
  extern __shared__ __align__(16) uint8_t row_smem[];   // [hidden/2] values, [hidden/16] scales
  __shared__ int s_owner[32], s_dest[32];
  __shared__ float s_gs[32];
  const int token = blockIdx.x;
  const int kblocks = p.hidden >> 4;
  uint8_t* s_q = row_smem;
  uint8_t* s_sf = row_smem + (p.hidden >> 1);
  if (threadIdx.x < 32) {
    const int k = threadIdx.x;
    int owner = -1, dest = 0;
    float gs = 0.0f;
    if (k < p.topk) {
      const long long entry = (long long)token * p.topk + k;
      const int e = __ldg(p.ids + entry);
      if (e >= 0 && e < p.experts_total) {
        dest = __ldg(p.send_base + e) + __ldg(p.rank_in_group + entry);
        if (dest >= 0 && dest < p.rows_cap) {
          owner = e / p.experts_local;
          gs = __ldg(p.gs + e);
          p.row_weight[owner][dest] = __ldg(p.weights + entry);
          if (p.row_dest[owner]) p.row_dest[owner][dest] = (p.rank << 26) | (int)entry;
          p.pair_row[entry] = dest;
        } else {
          atomicOr(p.status, kStatusEpOverflow);
          p.pair_row[entry] = -1;
        }
      } else {
        p.pair_row[entry] = -1;
      }
    }
    s_owner[k] = owner;
    s_dest[k] = dest;
    s_gs[k] = gs;
  }
  __syncthreads();
  if (p.row_next[0] && (int)threadIdx.x < p.topk) {
    // Same-rank pre-sum: the token's rows on one owner form a chain in pair order.  The first
    // one keeps its destination code (the owner sends the chain's sum there); the others are
    // marked absorbed on the owner (-2) and left out of this rank's final sum.
    const int k = threadIdx.x, owner = s_owner[k];
    if (owner >= 0) {
      int next = -1;
      bool first = true;
      for (int j = 0; j < p.topk; ++j) {
        if (j == k || s_owner[j] != owner) continue;
        if (j < k) first = false;
        else if (next < 0) next = s_dest[j];
      }
      const int dest = s_dest[k];
      p.row_next[owner][dest] = next;
      if (!first) {
        p.row_dest[owner][dest] = -2;
        p.pair_row[(long long)token * p.topk + k] = -2;
      }
    }
  }
  float have_gs = -1.0f;
  for (int k = 0; k < p.topk; ++k) {          // block-uniform control flow throughout
    const int owner = s_owner[k];
    if (owner < 0) continue;
    const float gs = s_gs[k];
    if (gs != have_gs) {
      if (have_gs >= 0.0f) {                  // earlier copies still read the row: let them finish
        if (threadIdx.x == 0) bulk_wait_group_read0();
        __syncthreads();
      }
      for (int kb = threadIdx.x; kb < kblocks; kb += blockDim.x) {
        float v[16];
        load16_bf16(p.tokens + (size_t)token * p.hidden + kb * 16, v);
        uint2 q8;
        uint32_t sfb;
        quantize_16(v, gs, q8, sfb);
        *reinterpret_cast<uint2*>(s_q + kb * 8) = q8;
        s_sf[kb] = (uint8_t)sfb;
      }
      fence_proxy_async_smem();
      __syncthreads();
      have_gs = gs;
    }
    if (threadIdx.x == 0) {
      const int dest = s_dest[k];
      bulk_store_1d(p.q[owner] + (size_t)dest * (p.hidden >> 1), smem_u32(s_q), (uint32_t)(p.hidden >> 1));
      bulk_store_1d(p.sf[owner] + (size_t)dest * kblocks, smem_u32(s_sf), (uint32_t)kblocks);
      bulk_commit_group();
    }
  }
  // the block may retire once the copies have read the row; the writes themselves are complete
  // when the grid is, which is what the next operation in the stream (the barrier) waits for
  if (threadIdx.x == 0) bulk_wait_group_read0();
  // only the first warp stored to other GPUs with plain stores (a system fence in every thread
  // was the kernel's largest stall under the profiler)
  if (threadIdx.x < 32) __threadfence_system();
}

// ---- combine ---------------------------------------------------------------------------------
struct EpCombineParams {
  const __nv_bfloat16* y[kMaxPeers];   // per rank: (rows_cap, hidden), routing weight applied
  const int* ids;                      // (tokens, topk)
  const int* pair_row;                 // (tokens, topk)
  __nv_bfloat16* out;                  // (tokens, hidden)
  int tokens, hidden, topk, experts_total, experts_local, rows_cap;
};

__global__ void __launch_bounds__(256) ep_combine_kernel(const EpCombineParams p) {
  const int vecs = p.hidden >> 3;
  const long long unit = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long token = unit / vecs;
  const int vc = (int)(unit - token * vecs);
  if (token >= p.tokens) return;
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (int k = 0; k < p.topk; ++k) {
    const long long entry = token * p.topk + k;
    const int e = __ldg(p.ids + entry);
    const int row = __ldg(p.pair_row + entry);
    if (e < 0 || e >= p.experts_total || row < 0 || row >= p.rows_cap) continue;
    const __nv_bfloat16* src = p.y[e / p.experts_local] + (size_t)row * p.hidden;
    const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(src) + vc);   // peer memory: L2 only
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(h[j]);
      acc[2 * j] = __fadd_rn(acc[2 * j], f.x);
      acc[2 * j + 1] = __fadd_rn(acc[2 * j + 1], f.y);
    }
  }
  uint32_t w[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    __nv_bfloat162 pr = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
    w[j] = *reinterpret_cast<uint32_t*>(&pr);
  }
  reinterpret_cast<uint4*>(p.out + (size_t)token * p.hidden)[vc] = make_uint4(w[0], w[1], w[2], w[3]);
}

// out[token] = bf16(sum over k, ascending, fp32) of y_pairs[token * topk + k]: the last step when
// the second GEMM has already delivered every pair's result row to the token's home rank.
// With pair_row, pairs marked negative (dropped on overflow, never delivered) are left out: their
// row of y_pairs still holds an earlier step's data.
__global__ void __launch_bounds__(256)
ep_sum_pairs_kernel(const __nv_bfloat16* __restrict__ y_pairs, const int* __restrict__ pair_row,
                    __nv_bfloat16* __restrict__ out, int tokens, int hidden, int topk) {
  // one CTA per token: which pairs count is looked up once, then every thread sums 8 columns at a
  // time with the loads of up to eight pairs issued before the first addition
  __shared__ int s_have[kMaxSumTopk];
  const long long token = blockIdx.x;
  if ((int)threadIdx.x < topk)
    s_have[threadIdx.x] = pair_row ? (__ldg(pair_row + token * topk + threadIdx.x) >= 0) : 1;
  __syncthreads();
  const int vecs = hidden >> 3;
  constexpr int kBatch = 8;
  const uint4* src = reinterpret_cast<const uint4*>(y_pairs + (size_t)token * topk * hidden);
  for (int vc = threadIdx.x; vc < vecs; vc += blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int k0 = 0; k0 < topk; k0 += kBatch) {
      uint4 raw[kBatch];
      bool have[kBatch];
#pragma unroll
      for (int j = 0; j < kBatch; ++j) {
        have[j] = k0 + j < topk && s_have[k0 + j];
        if (have[j]) raw[j] = __ldcg(src + (size_t)(k0 + j) * vecs + vc);
      }
#pragma unroll
      for (int j = 0; j < kBatch; ++j) {
        if (!have[j]) continue;
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[j]);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(h[i]);
          acc[2 * i] = __fadd_rn(acc[2 * i], f.x);
          acc[2 * i + 1] = __fadd_rn(acc[2 * i + 1], f.y);
        }
      }
    }
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      __nv_bfloat162 pr = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
      w[j] = *reinterpret_cast<uint32_t*>(&pr);
    }
    reinterpret_cast<uint4*>(out + (size_t)token * hidden)[vc] = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// ---- same-rank pre-sum ------------------------------------------------------------------------
// After the second GEMM has stored its rows locally: one CTA per local row that heads a chain
// (row_dest >= 0) adds the chain's rows in fp32, in chain order, rounds once to bf16 and writes
// the sum into the home rank's recv_y at the row the code names.  A token's k experts sit on
// about 5.3 of 8 ranks under uniform routing, so a third fewer rows cross NVLink than when
// every row is scattered by the GEMM's epilogue; the price is that the transfer no longer
// overlaps the GEMM, and one more rounding per rank the token visits.
struct EpPresumParams {
  const __nv_bfloat16* y;        // (rows, hidden) this rank's results, routing weight applied
  const int* row_dest;           // (rows)
  const int* row_next;           // (rows)
  uint8_t* dest[kMaxPeers];      // every rank's recv_y
  uint32_t* status;
  int rows, hidden, dest_count, dest_rows;
};

__global__ void __launch_bounds__(256) ep_presum_push_kernel(const EpPresumParams p) {
  const int row = blockIdx.x;
  const int code = __ldg(p.row_dest + row);
  if (code < 0) return;                                   // not a chain head (uniform over the CTA)
  const int drank = code >> 26, drow = code & 0x03ffffff;
  if (drank >= p.dest_count || drow >= p.dest_rows) {     // never turned into an address
    if (threadIdx.x == 0) atomicOr(p.status, 0x00C00000u);
    return;
  }
  __shared__ int s_chain[kMaxSumTopk];
  __shared__ int s_len;
  if (threadIdx.x == 0) {
    int n = 0, r = row;
    while (r >= 0 && r < p.rows && n < kMaxSumTopk) {     // bounded: a broken link cannot loop
      s_chain[n++] = r;
      r = __ldg(p.row_next + r);
    }
    s_len = n;
  }
  __syncthreads();
  const int len = s_len, vecs = p.hidden >> 3;
  uint4* dst = reinterpret_cast<uint4*>(p.dest[drank] + (size_t)drow * p.hidden * 2);
  for (int vc = threadIdx.x; vc < vecs; vc += blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int i = 0; i < len; ++i) {
      const uint4 raw = __ldg(reinterpret_cast<const uint4*>(p.y + (size_t)s_chain[i] * p.hidden) + vc);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        acc[2 * j] = __fadd_rn(acc[2 * j], f.x);
        acc[2 * j + 1] = __fadd_rn(acc[2 * j + 1], f.y);
      }
    }
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      __nv_bfloat162 pr = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
      w[j] = *reinterpret_cast<uint32_t*>(&pr);
    }
    dst[vc] = make_uint4(w[0], w[1], w[2], w[3]);
  }
  // the rows went to other GPUs: make them visible before the grid's completion is signalled
  __threadfence_system();
}

static int check_world(int world, int experts_total) {
  if (world < 1 || world > kMaxPeers)
    return fail(MSC_ERR_UNSUPPORTED, "world=%d must be in [1, %d]", world, kMaxPeers);
  if (experts_total <= 0 || experts_total % world)
    return fail(MSC_ERR_BAD_ARG, "%d experts do not split over %d ranks", experts_total, world);
  return MSC_OK;
}

}  // namespace msc

extern "C" {

int msc_peer_alloc(size_t bytes, void** ptr, void* handle64) {
  if (!ptr || !handle64 || bytes == 0) return msc::fail(MSC_ERR_BAD_ARG, "NULL pointer or zero size");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  void* d = nullptr;
  MSC_CUDA_OK(cudaMalloc(&d, bytes));
  cudaIpcMemHandle_t h;
  const cudaError_t e = cudaIpcGetMemHandle(&h, d);
  if (e != cudaSuccess) {
    cudaFree(d);
    return msc::fail(MSC_ERR_CUDA, "cudaIpcGetMemHandle: %s", cudaGetErrorString(e));
  }
  memcpy(handle64, &h, 64);
  *ptr = d;
  return MSC_OK;
}

int msc_peer_open(const void* handle64, void** ptr) {
  if (!handle64 || !ptr) return msc::fail(MSC_ERR_BAD_ARG, "NULL pointer");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void* d = nullptr;
  MSC_CUDA_OK(cudaIpcOpenMemHandle(&d, h, cudaIpcMemLazyEnablePeerAccess));
  *ptr = d;
  return MSC_OK;
}

int msc_peer_close(void* ptr) {
  if (!ptr) return msc::fail(MSC_ERR_BAD_ARG, "NULL pointer");
  MSC_CUDA_OK(cudaIpcCloseMemHandle(ptr));
  return MSC_OK;
}

int msc_peer_free(void* ptr) {
  if (!ptr) return msc::fail(MSC_ERR_BAD_ARG, "NULL pointer");
  MSC_CUDA_OK(cudaFree(ptr));
  return MSC_OK;
}

int msc_ep_offsets(const int32_t* counts_all, int world, int rank, int experts_total, int rows_cap,
                   int32_t* send_base, int32_t* group_rows, int32_t* group_offsets,
                   int32_t* total_rows, const int32_t* wait_flags, int wait_slot, int wait_epoch,
                   void* stream) {
  if (!counts_all || !send_base || !group_rows || !group_offsets || !total_rows)
    return msc::fail(MSC_ERR_BAD_ARG, "NULL pointer");
  int rc = msc::check_world(world, experts_total);
  if (rc) return rc;
  if (rank < 0 || rank >= world) return msc::fail(MSC_ERR_BAD_ARG, "rank=%d outside [0, %d)", rank, world);
  if (experts_total > 8192) return msc::fail(MSC_ERR_UNSUPPORTED, "experts_total=%d exceeds 8192", experts_total);
  if (rows_cap <= 0 || rows_cap % 128) return msc::fail(MSC_ERR_BAD_ARG, "rows_cap=%d must be a positive multiple of 128", rows_cap);
  if (wait_flags && (wait_slot < 0 || wait_slot >= msc::kFlagSlots))
    return msc::fail(MSC_ERR_BAD_ARG, "slot=%d outside [0, %d)", wait_slot, msc::kFlagSlots);
  uint32_t* status = reinterpret_cast<uint32_t*>(msc::status_word());
  if (!status) return MSC_ERR_CUDA;
  msc::ep_offsets_kernel<<<1, 256, experts_total * sizeof(int), static_cast<cudaStream_t>(stream)>>>(
      counts_all, world, rank, experts_total, experts_total / world, rows_cap, send_base, group_rows,
      group_offsets, total_rows, status, wait_flags, wait_slot, wait_epoch);
  MSC_CUDA_OK(cudaGetLastError());
  return MSC_OK;
}

int msc_ep_dispatch_quantize(const void* tokens_bf16, const int32_t* ids, const float* weights,
                             const int32_t* rank_in_group, const int32_t* send_base,
                             const float* input_gs, int tokens, int hidden, int topk,
                             int experts_total, int world, void* const* peer_a_q,
                             void* const* peer_sf_rows, float* const* peer_row_weight,
                             int32_t* const* peer_row_dest, int32_t* const* peer_row_next, int rank,
                             int rows_cap, int32_t* pair_row, void* stream) {
  if (!tokens_bf16 || !ids || !weights || !rank_in_group || !send_base || !input_gs || !peer_a_q ||
      !peer_sf_rows || !peer_row_weight || !pair_row)
    return msc::fail(MSC_ERR_BAD_ARG, "NULL pointer");
  int rc = msc::check_world(world, experts_total);
  if (rc) return rc;
  if (tokens <= 0 || topk <= 0) return msc::fail(MSC_ERR_BAD_ARG, "sizes must be positive");
  if (hidden <= 0 || hidden % 64) return msc::fail(MSC_ERR_BAD_ARG, "hidden=%d must be a multiple of 64", hidden);
  if (rows_cap <= 0 || rows_cap % 128) return msc::fail(MSC_ERR_BAD_ARG, "rows_cap=%d must be a positive multiple of 128", rows_cap);
  if (rank < 0 || rank >= world) return msc::fail(MSC_ERR_BAD_ARG, "rank=%d outside [0, %d)", rank, world);
  if ((long long)tokens * topk > 0x03ffffffLL)
    return msc::fail(MSC_ERR_UNSUPPORTED, "tokens * topk exceeds the 26 bits of a row destination code");
  if (peer_row_next && !peer_row_dest) return msc::fail(MSC_ERR_BAD_ARG, "row_next needs row_dest");
  if (peer_row_next && !(hidden % 256 == 0 && topk <= 32 && hidden <= 65536))
    return msc::fail(MSC_ERR_UNSUPPORTED, "the pre-summed combine needs hidden %% 256 == 0, hidden <= 65536, topk <= 32");
  msc::EpDispatchParams p;
  p.tokens = static_cast<const __nv_bfloat16*>(tokens_bf16);
  p.ids = ids; p.weights = weights; p.rank_in_group = rank_in_group; p.send_base = send_base;
  p.gs = input_gs; p.pair_row = pair_row;
  p.status = reinterpret_cast<uint32_t*>(msc::status_word());
  if (!p.status) return MSC_ERR_CUDA;
  for (int r = 0; r < msc::kMaxPeers; ++r) {
    const bool in = r < world;
    if (in && (!peer_a_q[r] || !peer_sf_rows[r] || !peer_row_weight[r]))
      return msc::fail(MSC_ERR_BAD_ARG, "NULL buffer for rank %d", r);
    p.q[r] = in ? static_cast<uint8_t*>(peer_a_q[r]) : nullptr;
    p.sf[r] = in ? static_cast<uint8_t*>(peer_sf_rows[r]) : nullptr;
    p.row_weight[r] = in ? peer_row_weight[r] : nullptr;
    p.row_dest[r] = (in && peer_row_dest) ? peer_row_dest[r] : nullptr;
    p.row_next[r] = (in && peer_row_next) ? peer_row_next[r] : nullptr;
    if (in && peer_row_next && !peer_row_next[r]) return msc::fail(MSC_ERR_BAD_ARG, "NULL row_next for rank %d", r);
    if (in && peer_row_dest && !peer_row_dest[r]) return msc::fail(MSC_ERR_BAD_ARG, "NULL row_dest for rank %d", r);
  }
  p.rank = rank;
  p.entries = tokens * topk; p.hidden = hidden; p.topk = topk;
  p.experts_total = experts_total; p.experts_local = experts_total / world; p.rows_cap = rows_cap;
  if (hidden % 256 == 0 && topk <= 32 && hidden <= 65536) {
    const int smem = hidden / 2 + hidden / 16;
    msc::ep_dispatch_bulk_kernel<<<(unsigned)tokens, 256, smem, static_cast<cudaStream_t>(stream)>>>(p);
    MSC_CUDA_OK(cudaGetLastError());
    return MSC_OK;
  }
  const long long units = (long long)tokens * (hidden / 16);
  const long long blocks = (units + 255) / 256;
  if (blocks > 0x7fffffffLL) return msc::fail(MSC_ERR_UNSUPPORTED, "problem too large for one launch");
  msc::ep_dispatch_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  MSC_CUDA_OK(cudaGetLastError());
  return MSC_OK;
}

int msc_ep_combine(const void* const* peer_y, const int32_t* ids, const int32_t* pair_row, void* out,
                   int tokens, int hidden, int topk, int experts_total, int world, int rows_cap,
                   void* stream) {
  if (!peer_y || !ids || !pair_row || !out) return msc::fail(MSC_ERR_BAD_ARG, "NULL pointer");
  int rc = msc::check_world(world, experts_total);
  if (rc) return rc;
  if (tokens <= 0 || topk <= 0) return msc::fail(MSC_ERR_BAD_ARG, "sizes must be positive");
  if (hidden <= 0 || hidden % 8) return msc::fail(MSC_ERR_BAD_ARG, "hidden=%d must be a multiple of 8", hidden);
  msc::EpCombineParams p;
  for (int r = 0; r < msc::kMaxPeers; ++r) {
    if (r < world && !peer_y[r]) return msc::fail(MSC_ERR_BAD_ARG, "NULL buffer for rank %d", r);
    p.y[r] = r < world ? static_cast<const __nv_bfloat16*>(peer_y[r]) : nullptr;
  }
  p.ids = ids; p.pair_row = pair_row; p.out = static_cast<__nv_bfloat16*>(out);
  p.tokens = tokens; p.hidden = hidden; p.topk = topk; p.experts_total = experts_total;
  p.experts_local = experts_total / world; p.rows_cap = rows_cap;
  const long long units = (long long)tokens * (hidden / 8);
  const long long blocks = (units + 255) / 256;
  if (blocks > 0x7fffffffLL) return msc::fail(MSC_ERR_UNSUPPORTED, "problem too large for one launch");
  msc::ep_combine_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  MSC_CUDA_OK(cudaGetLastError());
  return MSC_OK;
}

int msc_ep_signal(int32_t* const* peer_flags, int world, int rank, int slot, int epoch,
                  const int32_t* counts, int32_t* const* peer_counts_all, int experts_total,
                  void* stream) {
  if (!peer_flags) return msc::fail(MSC_ERR_BAD_ARG, "NULL pointer");
  if (world < 1 || world > msc::kMaxPeers)
    return msc::fail(MSC_ERR_UNSUPPORTED, "world=%d must be in [1, %d]", world, msc::kMaxPeers);
  if (rank < 0 || rank >= world) return msc::fail(MSC_ERR_BAD_ARG, "rank=%d outside [0, %d)", rank, world);
  if (slot < 0 || slot >= msc::kFlagSlots)
    return msc::fail(MSC_ERR_BAD_ARG, "slot=%d outside [0, %d)", slot, msc::kFlagSlots);
  if (counts && (!peer_counts_all || experts_total <= 0))
    return msc::fail(MSC_ERR_BAD_ARG, "counts need peer_counts_all and experts_total");
  msc::EpSignalParams p;
  for (int r = 0; r < msc::kMaxPeers; ++r) {
    if (r < world && (!peer_flags[r] || (counts && !peer_counts_all[r])))
      return msc::fail(MSC_ERR_BAD_ARG, "NULL buffer for rank %d", r);
    p.flags[r] = r < world ? peer_flags[r] : nullptr;
    p.counts_all[r] = (r < world && counts) ? peer_counts_all[r] : nullptr;
  }
  p.counts = counts;
  p.world = world; p.rank = rank; p.slot = slot; p.epoch = epoch; p.experts_total = experts_total;
  msc::ep_signal_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  MSC_CUDA_OK(cudaGetLastError());
  return MSC_OK;
}

int msc_ep_wait(const int32_t* flags, int world, int slot, int epoch, void* stream) {
  if (!flags) return msc::fail(MSC_ERR_BAD_ARG, "NULL pointer");
  if (world < 1 || world > msc::kMaxPeers)
    return msc::fail(MSC_ERR_UNSUPPORTED, "world=%d must be in [1, %d]", world, msc::kMaxPeers);
  if (slot < 0 || slot >= msc::kFlagSlots)
    return msc::fail(MSC_ERR_BAD_ARG, "slot=%d outside [0, %d)", slot, msc::kFlagSlots);
  uint32_t* status = reinterpret_cast<uint32_t*>(msc::status_word());
  if (!status) return MSC_ERR_CUDA;
  msc::ep_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(flags, world, slot, epoch, status);
  MSC_CUDA_OK(cudaGetLastError());
  return MSC_OK;
}

int msc_ep_presum_push(const void* y, const int32_t* row_dest, const int32_t* row_next,
                       void* const* dest_bases, int dest_count, int dest_rows, int rows, int hidden,
                       void* stream) {
  if (!y || !row_dest || !row_next || !dest_bases) return msc::fail(MSC_ERR_BAD_ARG, "NULL pointer");
  if (dest_count < 1 || dest_count > msc::kMaxPeers)
    return msc::fail(MSC_ERR_BAD_ARG, "dest_count=%d must be in [1, %d]", dest_count, msc::kMaxPeers);
  if (dest_rows <= 0 || dest_rows > 0x04000000) return msc::fail(MSC_ERR_BAD_ARG, "dest_rows out of range");
  if (rows <= 0) return msc::fail(MSC_ERR_BAD_ARG, "rows must be positive");
  if (hidden <= 0 || hidden % 8) return msc::fail(MSC_ERR_BAD_ARG, "hidden=%d must be a multiple of 8", hidden);
  msc::EpPresumParams p;
  p.y = static_cast<const __nv_bfloat16*>(y);
  p.row_dest = row_dest; p.row_next = row_next;
  for (int r = 0; r < msc::kMaxPeers; ++r) {
    if (r < dest_count && !dest_bases[r]) return msc::fail(MSC_ERR_BAD_ARG, "NULL destination %d", r);
    p.dest[r] = r < dest_count ? static_cast<uint8_t*>(dest_bases[r]) : nullptr;
  }
  p.status = reinterpret_cast<uint32_t*>(msc::status_word());
  if (!p.status) return MSC_ERR_CUDA;
  p.rows = rows; p.hidden = hidden; p.dest_count = dest_count; p.dest_rows = dest_rows;
  msc::ep_presum_push_kernel<<<(unsigned)rows, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  MSC_CUDA_OK(cudaGetLastError());
  return MSC_OK;
}

int msc_ep_sum_pairs(const void* y_pairs, const int32_t* pair_row, void* out, int tokens, int hidden,
                     int topk, void* stream) {
  if (!y_pairs || !out) return msc::fail(MSC_ERR_BAD_ARG, "NULL pointer");
  if (tokens <= 0 || topk <= 0) return msc::fail(MSC_ERR_BAD_ARG, "sizes must be positive");
  if (hidden <= 0 || hidden % 8) return msc::fail(MSC_ERR_BAD_ARG, "hidden=%d must be a multiple of 8", hidden);
  if (topk > msc::kMaxSumTopk) return msc::fail(MSC_ERR_UNSUPPORTED, "topk=%d exceeds %d", topk, msc::kMaxSumTopk);
  msc::ep_sum_pairs_kernel<<<(unsigned)tokens, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(y_pairs), pair_row, static_cast<__nv_bfloat16*>(out), tokens, hidden,
      topk);
  MSC_CUDA_OK(cudaGetLastError());
  return MSC_OK;
}

}  // extern "C"
