// Shared device/host helpers for the sm_100a kernel templates.
//
// Scope mapping used by every template (the reference tags buffers LOCAL / SHARED /
// GLOBAL in conductor/optimization/graph_analyzer.py:630-647):
//   LOCAL  -> registers (values never leave the thread that produced them)
//   SHARED -> shared memory or TMA-staged tiles (values exchanged inside one CTA)
//   GLOBAL -> HBM (cluster inputs and outputs)
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/conductor_b200.h"

namespace cdr {

// ---- error reporting (thread-local message read back by cdr_last_error) ----
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);

#define CDR_CUDA_TRY(expr)                                \
  do {                                                    \
    cudaError_t _e = (expr);                              \
    if (_e != cudaSuccess) return cdr::cuda_fail(_e, #expr); \
  } while (0)

inline int64_t numel(const cdr_tensor& t) {
  int64_t n = 1;
  for (int i = 0; i < t.rank; ++i) n *= t.shape[i];
  return n;
}

inline bool is_contiguous(const cdr_tensor& t) {
  int64_t expect = 1;
  for (int i = t.rank - 1; i >= 0; --i) {
    if (t.shape[i] != 1 && t.stride[i] != expect) return false;
    expect *= t.shape[i];
  }
  return true;
}

inline int dtype_size(int dt) {
  switch (dt) {
    case CDR_F32: return 4;
    case CDR_BF16: return 2;
    case CDR_F16: return 2;
    case CDR_I32: return 4;
    case CDR_I64: return 8;
    case CDR_BOOL: return 1;
    default: return 0;
  }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Number of SMs of the current device (cached per device).
int sm_count();
// Device pointer of the current device's status word (0 = ok; set by a kernel whose bounded
// wait gave up).  nullptr if it cannot be obtained; kernels accept that.
int* device_status_ptr();

// Per-template launchers (defined in the template's .cu file).
int launch_elementwise(const cdr_tensor* ins, int n_in, const cdr_tensor* outs, int n_out,
                       const cdr_ew_params* p, cudaStream_t stream);
int launch_row_reduce(const cdr_tensor* ins, int n_in, const cdr_tensor* outs, int n_out,
                      const cdr_reduce_params* p, cudaStream_t stream);
int full_reduce_workspace(const cdr_tensor* ins, int n_in, size_t* bytes);
// allow_runtime_instance = false keeps the call on the kernel compiled into the library (no
// NVRTC compile, no module load: nothing that allocates).
int launch_full_reduce(const cdr_tensor* ins, int n_in, const cdr_tensor* outs, int n_out,
                       const cdr_reduce_params* p, void* ws, size_t ws_bytes,
                       cudaStream_t stream, bool allow_runtime_instance = true);
// Shape / dtype / rank sanity of the tensor lists every entry point receives.
int check_lists(const cdr_tensor* ins, int n_in, const cdr_tensor* outs, int n_out);
void clear_error();
int col_sum_workspace(const cdr_tensor* ins, int n_in, const cdr_tensor* outs, int n_out, size_t* bytes);
int launch_col_sum(const cdr_tensor* ins, int n_in, const cdr_tensor* outs, int n_out, void* ws, size_t ws_bytes,
                   cudaStream_t stream);
int launch_softmax_fwd(const cdr_tensor* ins, int n_in, const cdr_tensor* outs, int n_out,
                       cudaStream_t stream);
int launch_softmax_bwd(const cdr_tensor* ins, int n_in, const cdr_tensor* outs, int n_out,
                       cudaStream_t stream);
int launch_gemm_epilogue(const cdr_tensor* ins, int n_in, const cdr_tensor* outs, int n_out,
                         const cdr_gemm_params* p, cudaStream_t stream);
int launch_strided_copy(const cdr_tensor* ins, int n_in, const cdr_tensor* outs, int n_out, cudaStream_t stream);
int launch_layer_norm(const cdr_tensor* ins, int n_in, const cdr_tensor* outs, int n_out, const cdr_norm_params* p,
                      cudaStream_t stream);
int launch_attention(const cdr_tensor* ins, int n_in, const cdr_tensor* outs, int n_out,
                     const cdr_attn_params* p, void* ws, size_t ws_bytes, cudaStream_t stream);
int attention_workspace(const cdr_tensor* ins, int n_in, size_t* bytes);

#ifdef __CUDACC__
// ---- 128-bit streaming global access -------------------------------------
// Cluster inputs and outputs are touched exactly once, so they bypass L1 and are
// marked evict-first in L2 (ld.global.cs / st.global.cs).
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  return __ldcs(reinterpret_cast<const uint4*>(p));
}
__device__ __forceinline__ void st_stream16(void* p, uint4 v) {
  __stcs(reinterpret_cast<uint4*>(p), v);
}
// Re-used operands (broadcast rows) go through the read-only path and stay in L1.
__device__ __forceinline__ uint4 ld_cached16(const void* p) {
  return __ldg(reinterpret_cast<const uint4*>(p));
}

// ---- dtype conversion ------------------------------------------------------
template <typename T> struct dtype_of;
template <> struct dtype_of<float> { static constexpr int value = CDR_F32; };
template <> struct dtype_of<__nv_bfloat16> { static constexpr int value = CDR_BF16; };
template <> struct dtype_of<__half> { static constexpr int value = CDR_F16; };

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }

// Round an fp32 value to the precision of `dt` (round-to-nearest-even) and return it
// as fp32: the value an eager low-precision op would have stored.
__device__ __forceinline__ float round_to_dtype(float v, int dt) {
  if (dt == CDR_BF16) return __bfloat162float(__float2bfloat16_rn(v));
  if (dt == CDR_F16) return __half2float(__float2half_rn(v));
  return v;
}
template <typename T> __device__ __forceinline__ float round_as(float v) {
  return to_f32<T>(from_f32<T>(v));
}

// Unpack a 16-byte register quad into N fp32 values (N = 16 / sizeof(T)).
template <typename T> struct Pack16;
template <> struct Pack16<float> {
  static constexpr int N = 4;
  __device__ __forceinline__ static void unpack(uint4 q, float* f) {
    f[0] = __uint_as_float(q.x); f[1] = __uint_as_float(q.y);
    f[2] = __uint_as_float(q.z); f[3] = __uint_as_float(q.w);
  }
  __device__ __forceinline__ static uint4 pack(const float* f) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]),
                      __float_as_uint(f[3]));
  }
};
template <> struct Pack16<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ __forceinline__ static void unpack(uint4 q, float* f) {
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      // a bf16 is the upper half of an fp32: widen with shifts, no cvt needed
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  __device__ __forceinline__ static uint4 pack(const float* f) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
};
template <> struct Pack16<__half> {
  static constexpr int N = 8;
  __device__ __forceinline__ static void unpack(uint4 q, float* f) {
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
      float2 v = __half22float2(h);
      f[2 * i] = v.x; f[2 * i + 1] = v.y;
    }
  }
  __device__ __forceinline__ static uint4 pack(const float* f) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __half2 h = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
};

// ---- warp / CTA reductions (warp shuffles, then one shared-memory hop) ------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
#endif  // __CUDACC__

}  // namespace cdr
