// Kernel activity records from CUPTI behind a flat C interface.
//
// The reference times kernels with the `cupti-python` package: its tracer registers buffer
// callbacks, enables CONCURRENT_KERNEL activity, runs the kernels, flushes, and reads one record
// per launch (src/mosaicist/bench/cupti_trace.py:51-80).  Where that package is not installed,
// the Python package next to this file offers the same five calls on top of this library, which
// talks to libcupti directly.  CUPTI invokes the buffer callbacks on its own threads, so records
// are copied into a vector here and handed to Python only when it asks.
#include <cupti.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>
#include <string>
#include <vector>

namespace {

struct Record {
  std::string name;
  uint64_t start, end;
  int32_t grid[3], block[3], cluster[3];
  int32_t dynamic_smem, static_smem, registers, local_mem;
  uint32_t kind;
};

std::mutex g_mu;
std::vector<Record> g_records;
size_t g_buffer_bytes = 8u << 20;
bool g_registered = false;
char g_error[256] = "";

int fail(CUptiResult r, const char* what) {
  const char* msg = nullptr;
  cuptiGetResultString(r, &msg);
  snprintf(g_error, sizeof(g_error), "%s: %s", what, msg ? msg : "unknown CUPTI error");
  return -1;
}

void CUPTIAPI buffer_requested(uint8_t** buffer, size_t* size, size_t* max_records) {
  void* p = nullptr;
  if (posix_memalign(&p, 8, g_buffer_bytes) != 0) p = nullptr;
  *buffer = static_cast<uint8_t*>(p);
  *size = p ? g_buffer_bytes : 0;
  *max_records = 0;
}

void CUPTIAPI buffer_completed(CUcontext, uint32_t, uint8_t* buffer, size_t, size_t valid) {
  CUpti_Activity* rec = nullptr;
  std::vector<Record> local;
  while (valid > 0 && cuptiActivityGetNextRecord(buffer, valid, &rec) == CUPTI_SUCCESS) {
    if (rec->kind == CUPTI_ACTIVITY_KIND_CONCURRENT_KERNEL || rec->kind == CUPTI_ACTIVITY_KIND_KERNEL) {
      const CUpti_ActivityKernel9* k = reinterpret_cast<const CUpti_ActivityKernel9*>(rec);
      Record r;
      r.name = k->name ? k->name : "";
      r.start = k->start;
      r.end = k->end;
      r.grid[0] = k->gridX; r.grid[1] = k->gridY; r.grid[2] = k->gridZ;
      r.block[0] = k->blockX; r.block[1] = k->blockY; r.block[2] = k->blockZ;
      r.cluster[0] = (int32_t)k->clusterX; r.cluster[1] = (int32_t)k->clusterY; r.cluster[2] = (int32_t)k->clusterZ;
      r.dynamic_smem = k->dynamicSharedMemory;
      r.static_smem = k->staticSharedMemory;
      r.registers = k->registersPerThread;
      r.local_mem = (int32_t)k->localMemoryPerThread;
      r.kind = (uint32_t)rec->kind;
      local.push_back(std::move(r));
    }
  }
  free(buffer);
  std::lock_guard<std::mutex> lock(g_mu);
  for (auto& r : local) g_records.push_back(std::move(r));
}

}  // namespace

extern "C" {

const char* msc_cupti_last_error(void) { return g_error; }

// Registers the buffer callbacks (once per process); later calls only update the buffer size.
int msc_cupti_register(size_t buffer_bytes) {
  if (buffer_bytes >= (64u << 10)) g_buffer_bytes = buffer_bytes;
  if (g_registered) return 0;
  CUptiResult r = cuptiActivityRegisterCallbacks(buffer_requested, buffer_completed);
  if (r != CUPTI_SUCCESS) return fail(r, "cuptiActivityRegisterCallbacks");
  g_registered = true;
  return 0;
}

int msc_cupti_enable(uint32_t kind) {
  CUptiResult r = cuptiActivityEnable(static_cast<CUpti_ActivityKind>(kind));
  return r == CUPTI_SUCCESS ? 0 : fail(r, "cuptiActivityEnable");
}

int msc_cupti_disable(uint32_t kind) {
  CUptiResult r = cuptiActivityDisable(static_cast<CUpti_ActivityKind>(kind));
  return r == CUPTI_SUCCESS ? 0 : fail(r, "cuptiActivityDisable");
}

int msc_cupti_flush(uint32_t flag) {
  CUptiResult r = cuptiActivityFlushAll(flag);
  return r == CUPTI_SUCCESS ? 0 : fail(r, "cuptiActivityFlushAll");
}

uint32_t msc_cupti_kind_concurrent_kernel(void) { return (uint32_t)CUPTI_ACTIVITY_KIND_CONCURRENT_KERNEL; }
uint32_t msc_cupti_kind_kernel(void) { return (uint32_t)CUPTI_ACTIVITY_KIND_KERNEL; }

size_t msc_cupti_count(void) {
  std::lock_guard<std::mutex> lock(g_mu);
  return g_records.size();
}

// Copies record i: name into name_out (NUL-terminated, at most name_cap bytes), start / end
// nanoseconds into times[2], grid / block / cluster / dynamic smem / static smem / registers /
// local memory per thread / kind into ints[13].  Returns 0, or -1 if i is out of range.
int msc_cupti_get(size_t i, char* name_out, size_t name_cap, uint64_t* times, int32_t* ints) {
  std::lock_guard<std::mutex> lock(g_mu);
  if (i >= g_records.size() || !name_out || !times || !ints || name_cap == 0) return -1;
  const Record& r = g_records[i];
  strncpy(name_out, r.name.c_str(), name_cap - 1);
  name_out[name_cap - 1] = 0;
  times[0] = r.start;
  times[1] = r.end;
  for (int d = 0; d < 3; ++d) {
    ints[d] = r.grid[d];
    ints[3 + d] = r.block[d];
    ints[6 + d] = r.cluster[d];
  }
  ints[9] = r.dynamic_smem;
  ints[10] = r.static_smem;
  ints[11] = r.registers;
  ints[12] = r.local_mem;
  return (int)r.kind;
}

void msc_cupti_clear(void) {
  std::lock_guard<std::mutex> lock(g_mu);
  g_records.clear();
}

}  // extern "C"
