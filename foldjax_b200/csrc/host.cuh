// Host-side plumbing shared by the translation units of libb200tri: error
// reporting, the device status word, TMA descriptor encoding (through the
// driver entry point, so the library does not link libcuda and still loads on
// a machine without a GPU), and the workspace carve-up helper.
#pragma once
#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "../../include/b200tri.h"

namespace b200 {

// Thread-local message behind b200tri_last_error().
void set_error(const char* fmt, ...);
const char* get_error();

// Address of this device's status word (global memory, zero = fine). Kernels
// record a bounded-wait timeout there.
int* device_status_word();

#define B200_CUDA_OK(expr)                                                              \
  do {                                                                                  \
    cudaError_t _e = (expr);                                                            \
    if (_e != cudaSuccess) {                                                            \
      b200::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, \
                      __LINE__);                                                        \
      return B200TRI_ERR_CUDA;                                                          \
    }                                                                                   \
  } while (0)

#define B200_REQUIRE(cond, code, ...) \
  do {                                \
    if (!(cond)) {                    \
      b200::set_error(__VA_ARGS__);   \
      return (code);                  \
    }                                 \
  } while (0)

enum class Swz { None, B64, B128 };

// Encode a tiled tensor map over `rank` dimensions (innermost first).
// strides_bytes[i] is the byte stride of dimension i+1 (dimension 0 is dense).
int make_tmap(CUtensorMap* out, const void* base, CUtensorMapDataType dtype, int rank, const uint64_t* dims,
              const uint64_t* strides_bytes, const uint32_t* box, Swz swz);

// Carves aligned pieces out of a caller-provided workspace.
struct Carver {
  uint8_t* base;
  size_t off = 0;
  explicit Carver(void* p) : base(static_cast<uint8_t*>(p)) {}
  template <typename T>
  T* take(size_t count, size_t align = 1024) {
    off = (off + align - 1) / align * align;
    T* p = base ? reinterpret_cast<T*>(base + off) : nullptr;
    off += count * sizeof(T);
    return p;
  }
  size_t total() const { return (off + 1023) / 1024 * 1024; }
};

inline int round_up(int x, int m) { return (x + m - 1) / m * m; }

// SMs the persistent kernels of the current device may use (its SM count, or the limit
// set for that device with b200tri_set_sm_limit).
int sm_count();
// While one of these lives, sm_count() on this host thread returns `keep` SMs fewer: the
// context-parallel ops leave room beside a persistent kernel for the small NCCL kernels that
// carry their tokens (a kernel that fills every SM would hold them back until it ends).
struct SmReserve {
  int before;
  explicit SmReserve(int keep);
  ~SmReserve();
};

// Raises a kernel's dynamic shared-memory limit, once per (kernel, device); safe to call
// from several host threads (one per device under XLA).
int ensure_smem_limit(const void* kernel, int bytes);

// The two module-level ops for every shape / element type outside the tensor-core
// specialisation (generic.cu): other channel and head counts, float32 trunks.
size_t trimul_workspace_bytes_generic(int32_t n, int32_t c_z, int32_t c_hidden, int32_t dtype);
size_t triatt_workspace_bytes_generic(int32_t n, int32_t c_z, int32_t heads, int32_t head_dim);
int trimul_forward_generic(const b200tri_trimul_args* a, int c_z, int c_hidden, cudaStream_t stream);
int triatt_forward_generic(const b200tri_triatt_args* a, int c_z, cudaStream_t stream);

// out[M][N] = (x * gate?) @ w (+ bias) (sigmoid?) (+ res): fp32 activations, bf16 weights [K][N]
// (single_attention.cu; the single track's projections and transition use it).
int launch_linear_f32(const float* x, const float* gate, const void* w, const void* bias, int M, int K, int N,
                      int sigmoid, const float* res, float* out, cudaStream_t stream);

// Launch accounting and optional per-kernel event timing.
enum KernelId { K_TRIMUL_PROJECT = 0, K_TRIMUL_CONTRACT, K_TRIMUL_FINISH, K_TRIATT_PROJECT, K_TRIATT_CORE,
                K_TRIATT_FINISH, K_PAIR_TRANSITION, K_PAIR_BIAS, K_CP_EXCHANGE, K_CP_READY, K_CP_COPY, K_COUNT };
void count_launch(int n = 1);
bool timing_enabled();
struct TimedLaunch {  // brackets the launches made during its lifetime
  int id;
  cudaStream_t stream;
  cudaEvent_t start = nullptr;
  TimedLaunch(int id, cudaStream_t stream, bool may_time = true);
  ~TimedLaunch();
};

}  // namespace b200
