// Library runtime: error text, device status word, TMA descriptor encoding.
#include <stdarg.h>
#include <stdio.h>

#include <string.h>

#include <atomic>
#include <mutex>
#include <utility>
#include <vector>

#include "host.cuh"
#include "tc.cuh"

namespace b200 {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}
const char* get_error() { return g_error; }

// One status word per device that loads the library.
__device__ int g_status_word = 0;

int* device_status_word() {
  constexpr int kMaxDev = 64;
  static int* cache[kMaxDev] = {nullptr};
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (!cache[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) return nullptr;
    cache[dev] = static_cast<int*>(p);
  }
  return cache[dev];
}

// Per-device settings: XLA drives every device from its own host thread, so a limit or
// the timing switch set with one device current must not leak to the others.
constexpr int kMaxDevices = 64;
static std::atomic<int> g_sm_limit[kMaxDevices];
static std::atomic<int> g_timing[kMaxDevices];

static int current_device_slot() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 0;
  return dev;
}

static int sm_count_device();

static thread_local int t_sm_reserve = 0;

SmReserve::SmReserve(int keep) : before(t_sm_reserve) { t_sm_reserve = keep > 0 ? keep : 0; }
SmReserve::~SmReserve() { t_sm_reserve = before; }

int sm_count() {
  int n = sm_count_device();
  const int lim = g_sm_limit[current_device_slot()].load(std::memory_order_relaxed);
  if (lim > 0 && lim < n) n = lim;
  return n - t_sm_reserve > 8 ? n - t_sm_reserve : n;
}

int ensure_smem_limit(const void* kernel, int bytes) {
  static std::mutex mu;
  static std::vector<std::pair<const void*, int>> done;
  const int dev = current_device_slot();
  std::lock_guard<std::mutex> lock(mu);
  for (const auto& e : done)
    if (e.first == kernel && e.second == dev) return B200TRI_OK;
  B200_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  done.emplace_back(kernel, dev);
  return B200TRI_OK;
}

static int sm_count_device() {
  constexpr int kMaxDev = 64;
  static int cache[kMaxDev] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return 148;
  if (!cache[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cache[dev] = n;
  }
  return cache[dev];
}

static std::atomic<uint64_t> g_launches{0};
static std::mutex g_timing_mu;
static std::vector<std::pair<cudaEvent_t, cudaEvent_t>> g_events[K_COUNT];
static const char* const kKernelNames[K_COUNT] = {"trimul_project", "trimul_contract", "trimul_finish",
                                                  "triatt_project", "triatt_core",     "triatt_finish",
                                                  "pair_transition", "pair_bias",      "cp_exchange",
                                                  "cp_ready",        "cp_copy"};

bool timing_enabled() { return g_timing[current_device_slot()].load(std::memory_order_relaxed) != 0; }

void count_launch(int n) { g_launches.fetch_add(static_cast<uint64_t>(n), std::memory_order_relaxed); }

TimedLaunch::TimedLaunch(int id_, cudaStream_t stream_, bool may_time) : id(id_), stream(stream_) {
  if (!may_time || !timing_enabled()) return;
  if (cudaEventCreate(&start) != cudaSuccess) {
    start = nullptr;
    return;
  }
  cudaEventRecord(start, stream);
}
TimedLaunch::~TimedLaunch() {
  if (!start) return;
  cudaEvent_t stop = nullptr;
  if (cudaEventCreate(&stop) != cudaSuccess) {
    cudaEventDestroy(start);
    return;
  }
  cudaEventRecord(stop, stream);
  std::lock_guard<std::mutex> lock(g_timing_mu);
  g_events[id].emplace_back(start, stop);
}

static PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  }
  return fn;
}

int make_tmap(CUtensorMap* out, const void* base, CUtensorMapDataType dtype, int rank, const uint64_t* dims,
              const uint64_t* strides_bytes, const uint32_t* box, Swz swz) {
  auto fn = encode_fn();
  B200_REQUIRE(fn != nullptr, B200TRI_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  B200_REQUIRE((reinterpret_cast<uintptr_t>(base) & 15) == 0, B200TRI_ERR_INVALID,
               "tensor base %p is not 16-byte aligned", base);
  for (int i = 0; i + 1 < rank; ++i)
    B200_REQUIRE((strides_bytes[i] & 15) == 0, B200TRI_ERR_INVALID,
                 "tensor stride %d (%llu bytes) is not a multiple of 16", i,
                 static_cast<unsigned long long>(strides_bytes[i]));
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUtensorMapSwizzle s = CU_TENSOR_MAP_SWIZZLE_NONE;
  if (swz == Swz::B64) s = CU_TENSOR_MAP_SWIZZLE_64B;
  if (swz == Swz::B128) s = CU_TENSOR_MAP_SWIZZLE_128B;
  CUresult r = fn(out, dtype, static_cast<cuuint32_t>(rank), const_cast<void*>(base), dims, strides_bytes, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, s, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  B200_REQUIRE(r == CUDA_SUCCESS, B200TRI_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return B200TRI_OK;
}

}  // namespace b200

namespace b200 {
// One warp waits on an mbarrier that nothing ever arrives at, through the same bounded wait
// every kernel of the library uses, with a caller-chosen limit.
__global__ void selftest_wait_kernel(long long limit_cycles, int* status) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    fence_barrier_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) mbar_wait_limited(&bar, 0, status, ST_TIMEOUT_SELFTEST, limit_cycles, 0u);
}
}  // namespace b200

extern "C" {

int b200tri_selftest_wait(int64_t limit_cycles, b200tri_stream_t stream) {
  using namespace b200;
  B200_REQUIRE(limit_cycles > 0 && limit_cycles <= 2000000000ll, B200TRI_ERR_INVALID,
               "selftest_wait: limit must be in (0, 2e9] cycles (got %lld)", static_cast<long long>(limit_cycles));
  int* status = device_status_word();
  B200_REQUIRE(status != nullptr, B200TRI_ERR_CUDA, "selftest_wait: no current CUDA device");
  count_launch();
  selftest_wait_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(limit_cycles, status);
  B200_CUDA_OK(cudaGetLastError());
  return B200TRI_OK;
}

int b200tri_version(void) { return 100; }

const char* b200tri_last_error(void) { return b200::get_error(); }

int b200tri_set_sm_limit(int32_t sms) {
  b200::g_sm_limit[b200::current_device_slot()].store(sms > 0 ? sms : 0);
  return B200TRI_OK;
}

uint64_t b200tri_launch_count(void) { return b200::g_launches.load(); }

int b200tri_timing_enable(int32_t on) {
  b200::g_timing[b200::current_device_slot()].store(on ? 1 : 0);
  return B200TRI_OK;
}

int b200tri_timing_reset(void) {
  std::lock_guard<std::mutex> lock(b200::g_timing_mu);
  for (auto& v : b200::g_events) {
    for (auto& e : v) {
      cudaEventDestroy(e.first);
      cudaEventDestroy(e.second);
    }
    v.clear();
  }
  return B200TRI_OK;
}

int b200tri_timing_read(const char* kernel, double* total_ms, int32_t* launches) {
  using namespace b200;
  B200_REQUIRE(kernel && total_ms && launches, B200TRI_ERR_INVALID, "timing_read: null argument");
  int id = -1;
  for (int i = 0; i < K_COUNT; ++i)
    if (strcmp(kernel, kKernelNames[i]) == 0) id = i;
  B200_REQUIRE(id >= 0, B200TRI_ERR_INVALID, "timing_read: unknown kernel name '%s'", kernel);
  B200_CUDA_OK(cudaDeviceSynchronize());
  std::lock_guard<std::mutex> lock(g_timing_mu);
  double sum = 0.0;
  for (auto& e : g_events[id]) {
    float ms = 0.f;
    B200_CUDA_OK(cudaEventElapsedTime(&ms, e.first, e.second));
    sum += ms;
  }
  *total_ms = sum;
  *launches = static_cast<int32_t>(g_events[id].size());
  return B200TRI_OK;
}

int b200tri_timing_list(const char* kernel, double* ms, int32_t capacity, int32_t* count) {
  using namespace b200;
  B200_REQUIRE(kernel && ms && count && capacity >= 0, B200TRI_ERR_INVALID, "timing_list: bad argument");
  int id = -1;
  for (int i = 0; i < K_COUNT; ++i)
    if (strcmp(kernel, kKernelNames[i]) == 0) id = i;
  B200_REQUIRE(id >= 0, B200TRI_ERR_INVALID, "timing_list: unknown kernel name '%s'", kernel);
  B200_CUDA_OK(cudaDeviceSynchronize());
  std::lock_guard<std::mutex> lock(g_timing_mu);
  int n = 0;
  for (auto& e : g_events[id]) {
    if (n >= capacity) break;
    float t = 0.f;
    B200_CUDA_OK(cudaEventElapsedTime(&t, e.first, e.second));
    ms[n++] = t;
  }
  *count = n;
  return B200TRI_OK;
}

int b200tri_device_status(void) {
  int* w = b200::device_status_word();
  if (!w) {
    b200::set_error("no CUDA device is current");
    return -1;
  }
  if (cudaDeviceSynchronize() != cudaSuccess) {
    b200::set_error("cudaDeviceSynchronize failed: %s", cudaGetErrorString(cudaGetLastError()));
    return -1;
  }
  int v = 0;
  if (cudaMemcpy(&v, w, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (v != 0) {
    int zero = 0;
    cudaMemcpy(w, &zero, sizeof(int), cudaMemcpyHostToDevice);
    b200::set_error("B200TRI_ERR_TIMEOUT: a kernel gave up on a bounded device wait (role code %d)", v);
  }
  return v;
}

}  // extern "C"
