// Error reporting, status word and tensor-map plumbing behind the C ABI.
#include "host_common.h"

#include <dlfcn.h>
#include <string.h>

#include <mutex>
#include <string>
#include <set>
#include <unordered_map>
#include <utility>

namespace msc {

static thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

// One status word per device that loads the library.  Kernels receive its address as an
// argument; a bounded wait that gives up stores (0x100 | wait id) here.
__device__ int g_status_word;

int* status_word() {
  static std::mutex mu;
  static int* cached[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (!cached[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) return nullptr;
    cached[dev] = static_cast<int*>(p);
  }
  return cached[dev];
}

int allow_dynamic_smem(const void* kernel, int bytes) {
  static std::mutex mu;
  static std::set<std::pair<const void*, int>> done;
  int dev = 0;
  MSC_CUDA_OK(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lock(mu);
  if (done.count({kernel, dev})) return MSC_OK;
  MSC_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  done.insert({kernel, dev});
  return MSC_OK;
}

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  if (!fn) fail(MSC_ERR_CUDA, "cuTensorMapEncodeTiled could not be resolved from the driver");
  return fn;
}

namespace {
struct TmapKey {
  const void* base;
  uint64_t rows, row_bytes;
  uint32_t box_rows;  // bits 31-28: 2 bf16 store map, 1 unswizzled scale map, 3 unswizzled 32-byte box, 0 operand map
  bool operator==(const TmapKey& o) const {
    return base == o.base && rows == o.rows && row_bytes == o.row_bytes && box_rows == o.box_rows;
  }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.base) * 0x9E3779B97F4A7C15ull;
    h ^= k.rows + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
    h ^= k.row_bytes + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
    return h ^ k.box_rows;
  }
};
int encode_tmap_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_bytes,
                   uint32_t box_rows, int flavour);
}  // namespace

// A tensor map only encodes address, shape and box, so one encoded for a buffer stays valid
// for any later buffer at the same address with the same shape: cache them, the driver call
// costs microseconds and the GEMM itself runs for about ten.
static std::mutex g_tmap_mu;
static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> g_tmap_cache;

void clear_tmap_cache() {
  std::lock_guard<std::mutex> lock(g_tmap_mu);
  g_tmap_cache.clear();
}

static int cached_tmap(CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_bytes,
                       uint32_t box_rows, int flavour) {
  std::mutex& mu = g_tmap_mu;
  auto& cache = g_tmap_cache;
  const TmapKey key{base, rows, row_bytes, box_rows | ((uint32_t)flavour << 28)};
  {
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *map = it->second;
      return MSC_OK;
    }
  }
  const int rc = encode_tmap_2d(map, base, rows, row_bytes, box_rows, flavour);
  if (rc == MSC_OK) {
    std::lock_guard<std::mutex> lock(mu);
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, *map);
  }
  return rc;
}

int make_tmap_bytes_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_bytes,
                       uint32_t box_rows) {
  return cached_tmap(map, base, rows, row_bytes, box_rows, 0);
}

int make_tmap_bf16_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols,
                      uint32_t box_rows) {
  return cached_tmap(map, base, rows, cols * 2, box_rows, 2);
}

int make_tmap_sf_2d(CUtensorMap* map, const void* base, uint64_t rows128, uint32_t box_rows) {
  return cached_tmap(map, base, rows128, 128, box_rows, 1);
}

int make_tmap_narrow_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_bytes,
                        uint32_t box_rows) {
  return cached_tmap(map, base, rows, row_bytes, box_rows, 3);
}

namespace {
int encode_tmap_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_bytes,
                   uint32_t box_rows, int flavour) {
  const bool bf16 = flavour == 2;
  const bool swizzled = flavour == 0 || flavour == 2;
  const cuuint32_t box_bytes = flavour == 3 ? 32u : 128u;
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return MSC_ERR_CUDA;
  if (reinterpret_cast<uintptr_t>(base) % 16 || row_bytes % 16)
    return fail(MSC_ERR_BAD_ARG, "operand base and row pitch must be 16-byte aligned");
  if (box_rows == 0 || box_rows > 256) return fail(MSC_ERR_BAD_ARG, "box rows out of range");
  // the box is 128 bytes wide (128 byte elements or 64 bf16 elements), 32 for the narrow flavour
  cuuint64_t dims[2] = {bf16 ? row_bytes / 2 : row_bytes, rows};
  cuuint64_t strides[1] = {row_bytes};
  cuuint32_t box[2] = {bf16 ? 64u : box_bytes, box_rows};
  cuuint32_t estr[2] = {1u, 1u};
  CUresult r = enc(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2,
                   const_cast<void*>(base), dims, strides,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzled ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(MSC_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return MSC_OK;
}
}  // namespace

int make_tmap_pitched_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_bytes,
                         uint64_t pitch_bytes, uint32_t box_rows) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return MSC_ERR_CUDA;
  if (reinterpret_cast<uintptr_t>(base) % 16 || pitch_bytes % 16 || row_bytes % 16)
    return fail(MSC_ERR_BAD_ARG, "matrix base, row length and pitch must be 16-byte aligned");
  if (box_rows == 0 || box_rows > 256) return fail(MSC_ERR_BAD_ARG, "box rows out of range");
  cuuint64_t dims[2] = {row_bytes, rows};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {128u, box_rows};
  cuuint32_t estr[2] = {1u, 1u};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(MSC_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return MSC_OK;
}

int num_sms() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (!cached[dev]) cudaDeviceGetAttribute(&cached[dev], cudaDevAttrMultiProcessorCount, dev);
  return cached[dev];
}

}  // namespace msc

extern "C" {

int msc_version(void) { return 1; }

int msc_shutdown(void) {
  msc::clear_tmap_cache();
  return MSC_OK;
}

const char* msc_last_error(void) { return msc::g_err; }

const char* msc_ptx_path(void) {
  static std::string path;
  static std::once_flag once;
  std::call_once(once, [] {
    Dl_info info;
    if (dladdr(reinterpret_cast<void*>(&msc_version), &info) && info.dli_fname) {
      std::string so(info.dli_fname);
      size_t dot = so.rfind(".so");
      path = (dot == std::string::npos ? so : so.substr(0, dot)) + ".ptx";
    }
  });
  return path.c_str();
}

int msc_status_word_read(int* out) {
  if (!out) return msc::fail(MSC_ERR_BAD_ARG, "out is NULL");
  int* w = msc::status_word();
  if (!w) return msc::fail(MSC_ERR_CUDA, "status word unavailable on this device");
  MSC_CUDA_OK(cudaDeviceSynchronize());
  MSC_CUDA_OK(cudaMemcpy(out, w, sizeof(int), cudaMemcpyDeviceToHost));
  if (*out != 0) MSC_CUDA_OK(cudaMemset(w, 0, sizeof(int)));
  return MSC_OK;
}

}  // extern "C"
