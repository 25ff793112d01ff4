// MoE routing and token movement around the grouped GEMMs (all HBM-bound):
//   route_topk        softmax over experts, top-k, renormalised weights  (one warp per token)
//   plan              per-expert row counts, each (token, k) pair's rank inside its expert in
//                     token order, and the 128-row-aligned offsets of the expert groups
//   permute_quantize  gathers each routed token row, quantises it to NVFP4 with its expert's
//                     global scale and writes it (values + tiled scales) at its group row
//   unpermute         out[token] = sum over k of the expert outputs of that token
// The reference has no routing or permutation code (its MoE takes per-expert padded batches,
// experiments/flashinfer-megamoe-sm100a/moe.py:47-79); these kernels produce exactly the
// row-concatenated, 128-aligned group layout the ragged GEMM entry points consume, with the
// per-row arithmetic of quantize_nvfp4 (nvfp4.py:39-57).
#include "host_common.h"
#include "ptx.cuh"
#include "quantize_common.cuh"

#include <mutex>

namespace msc {

constexpr int kMaxExpertsPerLane = 32;  // experts <= 1024

// ---- routing -----------------------------------------------------------------------------
// PER: register slots per lane (experts / 32 rounded up to 8 or 32); unused slots hold -inf / -1.
template <int PER>
__global__ void __launch_bounds__(128)
route_topk_kernel(const float* __restrict__ logits, int* __restrict__ ids, float* __restrict__ weights,
                  int tokens, int experts, int topk) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= tokens) return;
  const float* row = logits + (size_t)warp * experts;
  const int per = experts >> 5;
  float v[PER];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    v[i] = (i < per) ? __ldg(row + lane + 32 * i) : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.0f;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    v[i] = (i < per) ? expf(__fsub_rn(v[i], mx)) : -1.0f;   // -1 marks "not a candidate"
    if (i < per) sum = __fadd_rn(sum, v[i]);
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) sum = __fadd_rn(sum, __shfl_xor_sync(0xffffffffu, sum, o));

  float my_w = 0.0f;
  int my_id = 0;
  float wsum = 0.0f;
  for (int k = 0; k < topk; ++k) {
    float best = -1.0f;
    int best_i = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int idx = lane + 32 * i;
      if (v[i] > best || (v[i] == best && v[i] >= 0.0f && idx < best_i)) {
        best = v[i];
        best_i = idx;
      }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ob > best || (ob == best && oi < best_i)) {
        best = ob;
        best_i = oi;
      }
    }
    // the owner of the winning entry retires it (ties go to the lower expert index)
    if ((best_i & 31) == lane) {
#pragma unroll
      for (int i = 0; i < PER; ++i)
        if (i == (best_i >> 5)) v[i] = -1.0f;
    }
    const float pk = __fdiv_rn(best, sum);
    wsum = __fadd_rn(wsum, pk);
    if (lane == k) {
      my_w = pk;
      my_id = best_i;
    }
  }
  if (lane < topk) {
    ids[(size_t)warp * topk + lane] = my_id;
    weights[(size_t)warp * topk + lane] = __fdiv_rn(my_w, wsum);
  }
}

// ---- plan --------------------------------------------------------------------------------
// One block per local expert.  The block walks all (token, k) pairs in order, hands out ranks
// to the pairs routed to its expert (so rows inside a group keep token order) and records the
// group's row count.  The last block to finish (a ticket counter in `scratch`) turns the
// counts into 128-aligned group offsets and resets the ticket for the next call.
__global__ void __launch_bounds__(256)
moe_plan_kernel(const int* __restrict__ ids, int entries, int expert_first, int experts_local,
                int* __restrict__ rank, int* __restrict__ group_rows, int* __restrict__ group_offsets,
                int* __restrict__ total_rows, int* __restrict__ scratch) {
  constexpr int kSub = 4;                 // 1024-pair pieces handled between two block barriers
  __shared__ int warp_tot[2][kSub][8];
  __shared__ int is_last;
  const int e = blockIdx.x;
  const int want = expert_first + e;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const unsigned below = (1u << lane) - 1u;
  const bool vec = (reinterpret_cast<uintptr_t>(ids) & 15) == 0;
  int running = 0;
  // Each thread owns four consecutive pairs of every 1024-pair piece (one 16-byte load when the
  // piece is full) and a round covers kSub pieces, so the loads of a round are all in flight
  // together and a block barrier is paid once per 4096 pairs; the per-warp totals are
  // double-buffered.
  for (int base = 0, round = 0; base < entries; base += 1024 * kSub, ++round) {
    int4 v[kSub];
#pragma unroll
    for (int j = 0; j < kSub; ++j) {
      const int i0 = base + j * 1024 + threadIdx.x * 4;
      v[j] = make_int4(-1, -1, -1, -1);
      if (vec && i0 + 3 < entries) {
        v[j] = __ldg(reinterpret_cast<const int4*>(ids + i0));
      } else {
        if (i0 < entries) v[j].x = __ldg(ids + i0);
        if (i0 + 1 < entries) v[j].y = __ldg(ids + i0 + 1);
        if (i0 + 2 < entries) v[j].z = __ldg(ids + i0 + 2);
        if (i0 + 3 < entries) v[j].w = __ldg(ids + i0 + 3);
      }
    }
    unsigned b[kSub][4];
#pragma unroll
    for (int j = 0; j < kSub; ++j) {
      b[j][0] = __ballot_sync(0xffffffffu, v[j].x == want);
      b[j][1] = __ballot_sync(0xffffffffu, v[j].y == want);
      b[j][2] = __ballot_sync(0xffffffffu, v[j].z == want);
      b[j][3] = __ballot_sync(0xffffffffu, v[j].w == want);
      if (lane == 0)
        warp_tot[round & 1][j][warp] = __popc(b[j][0]) + __popc(b[j][1]) + __popc(b[j][2]) + __popc(b[j][3]);
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < kSub; ++j) {
      const int* tot = warp_tot[round & 1][j];
      int before = 0, total = 0;
#pragma unroll
      for (int w = 0; w < 8; ++w) {
        const int c = tot[w];
        if (w < warp) before += c;
        total += c;
      }
      const int i0 = base + j * 1024 + threadIdx.x * 4;
      const bool h0 = v[j].x == want, h1 = v[j].y == want, h2 = v[j].z == want, h3 = v[j].w == want;
      int r = running + before + __popc(b[j][0] & below) + __popc(b[j][1] & below) +
              __popc(b[j][2] & below) + __popc(b[j][3] & below);
      if (h0) rank[i0] = r;
      r += h0;
      if (h1) rank[i0 + 1] = r;
      r += h1;
      if (h2) rank[i0 + 2] = r;
      r += h2;
      if (h3) rank[i0 + 3] = r;
      running += total;
    }
  }
  if (threadIdx.x == 0) {
    group_rows[e] = running;
    __threadfence();
    const int ticket = atomicAdd(scratch, 1);
    is_last = (ticket == experts_local - 1);
  }
  __syncthreads();
  if (is_last) {
    // exclusive scan of the 128-aligned counts, 256 groups per round, by the whole block
    __threadfence();
    __shared__ int scan_tot[8];
    int carry = 0;
    for (int base = 0; base < experts_local; base += 256) {
      const int g = base + threadIdx.x;
      const int c = g < experts_local ? ((__ldcg(group_rows + g) + 127) & ~127) : 0;
      int incl = c;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += up;
      }
      if (lane == 31) scan_tot[warp] = incl;
      __syncthreads();
      int before = 0, total = 0;
#pragma unroll
      for (int w = 0; w < 8; ++w) {
        const int t = scan_tot[w];
        if (w < warp) before += t;
        total += t;
      }
      if (g < experts_local) group_offsets[g] = carry + before + incl - c;
      carry += total;
      __syncthreads();
    }
    if (threadIdx.x == 0) {
      *total_rows = carry;
      *scratch = 0;  // ready for the next call
    }
  }
}

// ---- dispatch: gather + quantise ---------------------------------------------------------
struct PermuteParams {
  const __nv_bfloat16* tokens;   // (tokens, hidden)
  const int* ids;                // (tokens, topk)
  const float* weights;          // (tokens, topk)
  const int* rank;               // (tokens, topk)
  const int* group_offsets;      // (experts_local)
  const float* gs;               // (experts_local) input global scale per expert
  uint8_t* q;                    // (rows_cap, hidden/2)
  uint8_t* sf;                   // tiled (rows_cap/128, hidden/64, 32, 16)
  uint8_t* sf_rows;              // (rows_cap, hidden/16) row-major staging for the scales, or null
  float* row_weight;             // (rows_cap)
  int* row_token;                // (rows_cap)
  int entries, hidden, topk, expert_first, experts_local;
};

constexpr int kMaxTopk = 64;   // pairs of one token the dispatch and combine kernels stage

// CTAs walk the tokens.  For each token the first warps look its pairs up once (expert, global
// scale, destination row); the CTA quantises the token's row into shared memory and one thread
// sends it to the row of every expert the token is routed to as one untiled bulk copy each
// (3.5 KB at hidden 7168) instead of hundreds of 8-byte stores.  The scale bytes go out either as
// words of the tiled layout (4 bytes every 512: one L2 transaction per word, which at top-8
// costs as much as everything else in the kernel) or, given a row-major staging buffer, as a
// second bulk copy per row that a re-tiling pass turns into the tiled layout afterwards.  Two
// row buffers alternate, so the copies of one token leave while the
// next is quantised.  The quantised bytes depend on the expert only through its global scale,
// so the row is re-quantised only when that scale differs from the one in shared memory (with
// one shared input scale a token is quantised once instead of topk times).
__global__ void __launch_bounds__(128) moe_permute_quantize_kernel(const PermuteParams p, int tokens) {
  extern __shared__ __align__(16) uint8_t row_smem[];   // 2 x ([hidden/2] values, [hidden/16] scales)
  __shared__ int s_dest[2][kMaxTopk];
  __shared__ float s_gs[2][kMaxTopk];
  const int kblocks = p.hidden >> 4;
  const int kwords = kblocks >> 2;
  const int row_bytes = ((p.hidden >> 1) + kblocks + 15) & ~15;   // bulk copies start 16-byte aligned
  int it = 0;
  for (long long token = blockIdx.x; token < tokens; token += gridDim.x, ++it) {
    const int buf = it & 1;
    uint8_t* s_q = row_smem + buf * row_bytes;
    uint8_t* s_sf = s_q + (p.hidden >> 1);
    // the copies of the token before last have read this buffer; the last token's may still run
    if (threadIdx.x == 0) bulk_wait_group_read1();
    if ((int)threadIdx.x < p.topk) {
      const int k = threadIdx.x;
      const int e = __ldg(p.ids + token * p.topk + k) - p.expert_first;
      int dest = -1;
      float g = 0.0f;
      if (e >= 0 && e < p.experts_local) {
        g = __ldg(p.gs + e);
        dest = __ldg(p.group_offsets + e) + __ldg(p.rank + token * p.topk + k);
        p.row_weight[dest] = __ldg(p.weights + token * p.topk + k);
        p.row_token[dest] = (int)token;
      }
      s_dest[buf][k] = dest;
      s_gs[buf][k] = g;
    }
    __syncthreads();
    float have_gs = -1.0f;   // global scales are positive: nothing is quantised yet
    for (int k = 0; k < p.topk; ++k) {            // CTA-uniform control flow throughout
      const int dest = s_dest[buf][k];
      if (dest < 0) continue;
      const float g = s_gs[buf][k];
      if (g != have_gs) {
        if (have_gs >= 0.0f) {                    // this token's earlier copies still read the row
          if (threadIdx.x == 0) {
            bulk_commit_group();
            bulk_wait_group_read0();
          }
          __syncthreads();
        }
        for (int kb = threadIdx.x; kb < kblocks; kb += blockDim.x) {
          float v[16];
          load16_bf16(p.tokens + (size_t)token * p.hidden + kb * 16, v);
          uint2 q8;
          uint32_t sfb;
          quantize_16(v, g, q8, sfb);
          *reinterpret_cast<uint2*>(s_q + kb * 8) = q8;
          s_sf[kb] = (uint8_t)sfb;
        }
        fence_proxy_async_smem();
        __syncthreads();
        have_gs = g;
      }
      if (threadIdx.x == 0) {
        bulk_store_1d(p.q + (size_t)dest * (p.hidden >> 1), smem_u32(s_q), (uint32_t)(p.hidden >> 1));
        if (p.sf_rows) bulk_store_1d(p.sf_rows + (size_t)dest * kblocks, smem_u32(s_sf), (uint32_t)kblocks);
      }
      if (!p.sf_rows)
        for (int w = threadIdx.x; w < kwords; w += blockDim.x)
          *reinterpret_cast<uint32_t*>(p.sf + tiled_sf_word(dest, w, kwords)) =
              reinterpret_cast<const uint32_t*>(s_sf)[w];
    }
    if (threadIdx.x == 0) bulk_commit_group();    // one group per token (empty ones count too)
  }
  if (threadIdx.x == 0) bulk_wait_group_read0();  // the rows are read before the CTA retires
}

// ---- combine -----------------------------------------------------------------------------
// One CTA per token: the rows holding the token's expert outputs are looked up once, then
// every thread sums 8 columns at a time over those rows, in the order of the token's pairs,
// with the loads of up to eight rows issued before the first addition.
__global__ void __launch_bounds__(256)
moe_unpermute_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ ids,
                     const int* __restrict__ rank, const int* __restrict__ group_offsets,
                     __nv_bfloat16* __restrict__ out, int tokens, int hidden, int topk,
                     int expert_first, int experts_local) {
  __shared__ int s_row[kMaxTopk];
  const long long token = blockIdx.x;
  if ((int)threadIdx.x < topk) {
    const long long entry = token * topk + threadIdx.x;
    const int e = __ldg(ids + entry) - expert_first;
    s_row[threadIdx.x] = (e < 0 || e >= experts_local) ? -1 : __ldg(group_offsets + e) + __ldg(rank + entry);
  }
  __syncthreads();
  const int vecs = hidden >> 3;  // 8 bf16 per thread and step
  constexpr int kBatch = 8;
  for (int vc = threadIdx.x; vc < vecs; vc += blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int k0 = 0; k0 < topk; k0 += kBatch) {
      uint4 raw[kBatch];
      bool have[kBatch];
#pragma unroll
      for (int j = 0; j < kBatch; ++j) {
        const int row = (k0 + j < topk) ? s_row[k0 + j] : -1;
        have[j] = row >= 0;
        if (have[j]) raw[j] = __ldg(reinterpret_cast<const uint4*>(y + (size_t)row * hidden) + vc);
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

static int launch_plan(const int32_t* ids, int entries, int expert_first, int experts_local,
                       int32_t* rank, int32_t* group_rows, int32_t* group_offsets,
                       int32_t* total_rows, int32_t* scratch, void* stream) {
  if (!ids || !rank || !group_rows || !group_offsets || !total_rows || !scratch)
    return fail(MSC_ERR_BAD_ARG, "NULL pointer");
  if (entries <= 0 || experts_local <= 0) return fail(MSC_ERR_BAD_ARG, "sizes must be positive");
  moe_plan_kernel<<<experts_local, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      ids, entries, expert_first, experts_local, rank, group_rows, group_offsets, total_rows, scratch);
  MSC_CUDA_OK(cudaGetLastError());
  return MSC_OK;
}

// ---- plan without caller-provided or allocated scratch ------------------------------------
// Some hosts of this library may not allocate device memory at the point where they plan a
// batch: a serving loop whose memory pool is frozen after start-up, a plugin called from a
// framework that owns every allocation, code running between the steps of a captured
// pipeline.  For them the ticket counter, and the row counts and total when the caller does
// not ask for them, live in this fixed array inside the library image.  Every device that
// loads the library carries these 4352 bytes until the process exits.
constexpr int kPlanStaticMaxExperts = 1024;
constexpr int kPlanStaticCountsAt = 64;   // [0] ticket, [1] total rows, [64...] row counts
static __device__ __align__(256) int g_plan_scratch[kPlanStaticCountsAt + kPlanStaticMaxExperts];

// Device address of g_plan_scratch on the current device.  In host code the symbol name is
// only a handle, never an address a kernel may be given; the address comes from the runtime,
// once per device, with that device current.
static int plan_scratch_address(int** out) {
  static std::mutex mu;
  static int* cached[64] = {nullptr};
  int dev = 0;
  MSC_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(MSC_ERR_UNSUPPORTED, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (!cached[dev]) {
    int* ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_plan_scratch);
    if (e != cudaSuccess || !ptr)
      return fail(MSC_ERR_CUDA, "cudaGetSymbolAddress(plan scratch): %s", cudaGetErrorString(e));
    cached[dev] = ptr;
  }
  *out = cached[dev];
  return MSC_OK;
}

}  // namespace msc

extern "C" {

int msc_moe_plan_noalloc(const int32_t* ids, int entries, int expert_first, int experts_local,
                         int32_t* rank, int32_t* group_rows, int32_t* group_offsets,
                         int32_t* total_rows, void* stream) {
  if (experts_local > msc::kPlanStaticMaxExperts)
    return msc::fail(MSC_ERR_BAD_ARG,
                     "experts_local=%d exceeds the %d experts the built-in scratch area holds; "
                     "use msc_moe_plan with caller-provided scratch",
                     experts_local, msc::kPlanStaticMaxExperts);
  // refuse bad arguments before anything is enqueued on the stream
  if (!ids || !rank || !group_offsets) return msc::fail(MSC_ERR_BAD_ARG, "NULL pointer");
  if (entries <= 0 || experts_local <= 0) return msc::fail(MSC_ERR_BAD_ARG, "sizes must be positive");
  int* scratch = nullptr;
  const int rc = msc::plan_scratch_address(&scratch);
  if (rc) return rc;
  // the ticket must be zero when the kernel starts, whatever an earlier call left behind
  MSC_CUDA_OK(cudaMemsetAsync(scratch, 0, sizeof(int), static_cast<cudaStream_t>(stream)));
  return msc::launch_plan(ids, entries, expert_first, experts_local, rank,
                          group_rows ? group_rows : scratch + msc::kPlanStaticCountsAt,
                          group_offsets, total_rows ? total_rows : scratch + 1, scratch, stream);
}

int msc_moe_route_topk(const float* logits, int32_t* ids, float* weights, int tokens, int experts,
                       int topk, void* stream) {
  if (!logits || !ids || !weights) return msc::fail(MSC_ERR_BAD_ARG, "NULL pointer");
  if (tokens <= 0) return msc::fail(MSC_ERR_BAD_ARG, "tokens must be positive");
  if (experts < 32 || experts > 32 * msc::kMaxExpertsPerLane || experts % 32)
    return msc::fail(MSC_ERR_UNSUPPORTED, "experts=%d must be a multiple of 32 in [32, 1024]", experts);
  if (topk < 1 || topk > 32 || topk > experts)
    return msc::fail(MSC_ERR_UNSUPPORTED, "topk=%d must be in [1, 32]", topk);
  const int blocks = (tokens + 3) / 4;
  if (experts <= 256)
    msc::route_topk_kernel<8><<<blocks, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        logits, ids, weights, tokens, experts, topk);
  else
    msc::route_topk_kernel<msc::kMaxExpertsPerLane><<<blocks, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        logits, ids, weights, tokens, experts, topk);
  MSC_CUDA_OK(cudaGetLastError());
  return MSC_OK;
}

int msc_moe_plan(const int32_t* ids, int entries, int expert_first, int experts_local,
                 int32_t* rank, int32_t* group_rows, int32_t* group_offsets, int32_t* total_rows,
                 int32_t* scratch, void* stream) {
  return msc::launch_plan(ids, entries, expert_first, experts_local, rank, group_rows,
                          group_offsets, total_rows, scratch, stream);
}

int msc_moe_permute_quantize(const void* tokens_bf16, const int32_t* ids, const float* weights,
                             const int32_t* rank, const int32_t* group_offsets,
                             const float* input_gs, int tokens, int hidden, int topk,
                             int expert_first, int experts_local, void* a_q, void* a_sf,
                             float* row_weight, int32_t* row_token, void* sf_rows, int rows_cap,
                             const int32_t* total_rows, void* stream) {
  if (!tokens_bf16 || !ids || !weights || !rank || !group_offsets || !input_gs || !a_q || !a_sf ||
      !row_weight || !row_token)
    return msc::fail(MSC_ERR_BAD_ARG, "NULL pointer");
  if (tokens <= 0 || topk <= 0 || experts_local <= 0) return msc::fail(MSC_ERR_BAD_ARG, "sizes must be positive");
  if (hidden <= 0 || hidden % 64) return msc::fail(MSC_ERR_BAD_ARG, "hidden=%d must be a multiple of 64", hidden);
  msc::PermuteParams p;
  p.tokens = static_cast<const __nv_bfloat16*>(tokens_bf16);
  p.ids = ids; p.weights = weights; p.rank = rank; p.group_offsets = group_offsets; p.gs = input_gs;
  p.q = static_cast<uint8_t*>(a_q); p.sf = static_cast<uint8_t*>(a_sf);
  p.row_weight = row_weight; p.row_token = row_token;
  // the staged form needs scale rows that bulk copies can carry (a multiple of 16 bytes)
  const bool staged = sf_rows != nullptr;
  if (staged) {
    if (hidden % 256) return msc::fail(MSC_ERR_BAD_ARG, "sf_rows needs hidden %% 256 == 0, got %d", hidden);
    if (rows_cap <= 0 || rows_cap % 128) return msc::fail(MSC_ERR_BAD_ARG, "rows_cap=%d must be a positive multiple of 128", rows_cap);
    if (reinterpret_cast<uintptr_t>(sf_rows) % 16 || reinterpret_cast<uintptr_t>(a_sf) % 16)
      return msc::fail(MSC_ERR_BAD_ARG, "sf_rows and a_sf must be 16-byte aligned");
  }
  p.sf_rows = static_cast<uint8_t*>(sf_rows);
  p.entries = tokens * topk; p.hidden = hidden; p.topk = topk;
  p.expert_first = expert_first; p.experts_local = experts_local;
  if (topk > msc::kMaxTopk) return msc::fail(MSC_ERR_UNSUPPORTED, "topk=%d exceeds %d", topk, msc::kMaxTopk);
  if (reinterpret_cast<uintptr_t>(a_q) % 16)
    return msc::fail(MSC_ERR_BAD_ARG, "a_q must be 16-byte aligned");
  const int smem = 2 * ((hidden / 2 + hidden / 16 + 15) & ~15);
  if (smem > 200 * 1024) return msc::fail(MSC_ERR_UNSUPPORTED, "hidden=%d: two rows do not fit in shared memory", hidden);
  if (smem > 48 * 1024)
    if (int rc = msc::allow_dynamic_smem(reinterpret_cast<const void*>(msc::moe_permute_quantize_kernel), 200 * 1024))
      return rc;
  // enough CTAs to fill every SM (16 x 128 threads), each walking its share of the tokens
  const int sms = msc::num_sms();
  if (sms <= 0) return msc::fail(MSC_ERR_CUDA, "could not query the SM count");
  const int grid = tokens < 16 * sms ? tokens : 16 * sms;
  msc::moe_permute_quantize_kernel<<<grid, 128, smem, static_cast<cudaStream_t>(stream)>>>(p, tokens);
  MSC_CUDA_OK(cudaGetLastError());
  if (staged)
    return msc::launch_sf_swizzle(sf_rows, a_sf, 1, rows_cap, hidden / 64, total_rows,
                                  static_cast<cudaStream_t>(stream));
  return MSC_OK;
}

int msc_moe_unpermute(const void* y, const int32_t* ids, const int32_t* rank,
                      const int32_t* group_offsets, void* out, int tokens, int hidden, int topk,
                      int expert_first, int experts_local, void* stream) {
  if (!y || !ids || !rank || !group_offsets || !out) return msc::fail(MSC_ERR_BAD_ARG, "NULL pointer");
  if (tokens <= 0 || topk <= 0 || experts_local <= 0) return msc::fail(MSC_ERR_BAD_ARG, "sizes must be positive");
  if (hidden <= 0 || hidden % 8) return msc::fail(MSC_ERR_BAD_ARG, "hidden=%d must be a multiple of 8", hidden);
  if (topk > msc::kMaxTopk) return msc::fail(MSC_ERR_UNSUPPORTED, "topk=%d exceeds %d", topk, msc::kMaxTopk);
  msc::moe_unpermute_kernel<<<(unsigned)tokens, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(y), ids, rank, group_offsets,
      static_cast<__nv_bfloat16*>(out), tokens, hidden, topk, expert_first, experts_local);
  MSC_CUDA_OK(cudaGetLastError());
  return MSC_OK;
}

}  // extern "C"
