// K3 -- row softmax, forward and backward, over the last dimension.
//
// Scalar definitions in the reference: three-pass forward
// choreo-op/softmax-gcu-only-test.co:14-32, online (running max / running sum)
// forward choreo-op/online-softmax-gcu-only-test.co:13-29, Jacobian backward
// choreo-op/softmaxbw-gcu-only-test.co:13-24.  The executed path is eager
// torch.softmax / torch._softmax_backward_data.
//
// HBM-bound, one pass over memory: a row is loaded once with 128-bit streaming loads
// and stays in registers (LOCAL scope) until its result is stored.
//   forward : every thread forms a partial (max m_t, sum s_t of exp(x - m_t)) over its
//             slice, partials are merged with the online-softmax recurrence
//             s = s_a * exp(m_a - m) + s_b * exp(m_b - m) through warp shuffles and one
//             shared-memory hop, then y = exp(x - m_t) * (exp(m_t - m) / s).
//   backward: dx = y * (g - sum(g * y)), the O(n) form of the reference's O(n^2) Jacobian
//             product.
// Per element exp(x - m) is ex2.approx((x - m) * log2(e)): relative error below 2e-6 for the
// arguments a softmax row produces (the fp32 bar is 1e-5), and 3 instructions instead of the
// ~15 of expf -- the accurate expf made this kernel issue-bound (78 % issue slots busy at 72 % of
// DRAM peak).  Per-thread and per-row quantities still use expf and IEEE division.
#include <math.h>

#include "cdr_common.cuh"

namespace cdr {
namespace {

struct SmArgs {
  const void* in0;  // forward: logits; backward: grad_out
  const void* in1;  // backward: y
  void* out;
  int64_t rows;
  int64_t cols;
};

struct MS { float m, s; };

__device__ __forceinline__ float exp_fast(float d) {   // exp(d) for d <= 0 (or -inf)
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(d * 1.4426950408889634f));
  return y;
}

__device__ __forceinline__ MS ms_merge(MS a, MS b) {
  const float m = fmaxf(a.m, b.m);
  // a side whose max is -inf holds no finite element: its sum is 0 and must not
  // produce exp(-inf - -inf) = NaN
  const float sa = (a.m == -INFINITY) ? 0.0f : a.s * expf(a.m - m);
  const float sb = (b.m == -INFINITY) ? 0.0f : b.s * expf(b.m - m);
  return MS{m, sa + sb};
}

template <int WIDTH>
__device__ __forceinline__ MS ms_shuffle_reduce(MS v) {
#pragma unroll
  for (int o = WIDTH / 2; o > 0; o >>= 1) {
    MS other{__shfl_xor_sync(0xffffffffu, v.m, o), __shfl_xor_sync(0xffffffffu, v.s, o)};
    v = ms_merge(v, other);
  }
  return v;
}
template <int WIDTH>
__device__ __forceinline__ float sum_shuffle_reduce(float v) {
#pragma unroll
  for (int o = WIDTH / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// TPR threads cooperate on one row; a CTA holds max(256, TPR) threads, i.e. 256/TPR rows.
template <typename T, int TPR, int VPT>
__global__ void __launch_bounds__((TPR > 256 ? TPR : 256)) softmax_fwd_kernel(const __grid_constant__ SmArgs a) {
  constexpr int V = Pack16<T>::N;
  constexpr int NT = TPR > 256 ? TPR : 256;
  constexpr int RPC = NT / TPR;                  // rows per CTA
  constexpr int WPR = TPR > 32 ? TPR / 32 : 1;   // warps per row
  __shared__ float sm_m[RPC][WPR], sm_s[RPC][WPR];

  const int tid = threadIdx.x;
  const int rloc = tid / TPR, t = tid % TPR;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * RPC + rloc;
  const bool live = row < a.rows;
  const int64_t vec_per_row = a.cols / V;
  const T* src = static_cast<const T*>(a.in0) + (live ? row : 0) * a.cols;

  float x[VPT][V];
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int64_t v = t + static_cast<int64_t>(j) * TPR;
    if (live && v < vec_per_row) {
      Pack16<T>::unpack(ld_stream16(src + v * V), x[j]);
    } else {
#pragma unroll
      for (int e = 0; e < V; ++e) x[j][e] = -INFINITY;
    }
  }

  float m_t = -INFINITY;
#pragma unroll
  for (int j = 0; j < VPT; ++j)
#pragma unroll
    for (int e = 0; e < V; ++e) m_t = fmaxf(m_t, x[j][e]);
  // a slice with no finite element (m_t == -inf) must contribute exp(-inf) = 0, not exp(NaN)
  const float m_sub = (m_t == -INFINITY) ? 0.0f : m_t;
  float s0 = 0.0f, s1 = 0.0f;
#pragma unroll
  for (int j = 0; j < VPT; ++j)
#pragma unroll
    for (int e = 0; e < V; e += 2) {
      const float e0 = exp_fast(x[j][e] - m_sub), e1 = exp_fast(x[j][e + 1] - m_sub);
      x[j][e] = e0;
      x[j][e + 1] = e1;
      s0 += e0;
      s1 += e1;
    }
  const float s_t = s0 + s1;

  MS ms = ms_shuffle_reduce<(TPR < 32 ? TPR : 32)>(MS{m_t, s_t});
  if (WPR > 1) {
    const int w = t >> 5;
    if ((t & 31) == 0) { sm_m[rloc][w] = ms.m; sm_s[rloc][w] = ms.s; }
    __syncthreads();
    MS acc{sm_m[rloc][0], sm_s[rloc][0]};
#pragma unroll
    for (int k = 1; k < WPR; ++k) acc = ms_merge(acc, MS{sm_m[rloc][k], sm_s[rloc][k]});
    ms = acc;
  }
  // rows with no finite element (all -inf) give 0/0 = NaN, as eager does
  // y = e * (exp(m_t - m) / s): one division per thread, one multiply per element
  const float factor = __fdiv_rn(m_t == -INFINITY ? 0.0f : expf(m_t - ms.m), ms.s);

  T* dst = static_cast<T*>(a.out) + (live ? row : 0) * a.cols;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int64_t v = t + static_cast<int64_t>(j) * TPR;
    if (live && v < vec_per_row) {
      float y[V];
#pragma unroll
      for (int e = 0; e < V; ++e) y[e] = x[j][e] * factor;
      st_stream16(dst + v * V, Pack16<T>::pack(y));
    }
  }
}

template <typename T, int TPR, int VPT>
__global__ void __launch_bounds__((TPR > 256 ? TPR : 256)) softmax_bwd_kernel(const __grid_constant__ SmArgs a) {
  constexpr int V = Pack16<T>::N;
  constexpr int NT = TPR > 256 ? TPR : 256;
  constexpr int RPC = NT / TPR;
  constexpr int WPR = TPR > 32 ? TPR / 32 : 1;
  __shared__ float sm_d[RPC][WPR];

  const int tid = threadIdx.x;
  const int rloc = tid / TPR, t = tid % TPR;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * RPC + rloc;
  const bool live = row < a.rows;
  const int64_t vec_per_row = a.cols / V;
  const int64_t off = (live ? row : 0) * a.cols;
  const T* gsrc = static_cast<const T*>(a.in0) + off;
  const T* ysrc = static_cast<const T*>(a.in1) + off;

  uint4 gq[VPT], yq[VPT];
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int64_t v = t + static_cast<int64_t>(j) * TPR;
    const bool ok = live && v < vec_per_row;
    gq[j] = ok ? ld_stream16(gsrc + v * V) : make_uint4(0, 0, 0, 0);
    yq[j] = ok ? ld_stream16(ysrc + v * V) : make_uint4(0, 0, 0, 0);
  }
  float g[VPT][V], y[VPT][V];
  float d0 = 0.0f, d1 = 0.0f;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    Pack16<T>::unpack(gq[j], g[j]);
    Pack16<T>::unpack(yq[j], y[j]);
#pragma unroll
    for (int e = 0; e < V; e += 2) {
      d0 = fmaf(g[j][e], y[j][e], d0);
      d1 = fmaf(g[j][e + 1], y[j][e + 1], d1);
    }
  }
  float dot = sum_shuffle_reduce<(TPR < 32 ? TPR : 32)>(d0 + d1);
  if (WPR > 1) {
    const int w = t >> 5;
    if ((t & 31) == 0) sm_d[rloc][w] = dot;
    __syncthreads();
    float acc = 0.0f;
#pragma unroll
    for (int k = 0; k < WPR; ++k) acc += sm_d[rloc][k];
    dot = acc;
  }
  T* dst = static_cast<T*>(a.out) + off;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int64_t v = t + static_cast<int64_t>(j) * TPR;
    if (live && v < vec_per_row) {
      float dx[V];
#pragma unroll
      for (int e = 0; e < V; ++e) dx[e] = (g[j][e] - dot) * y[j][e];
      st_stream16(dst + v * V, Pack16<T>::pack(dx));
    }
  }
}

// Any row length / alignment: one CTA per row, three passes over global memory (the
// row is served from L2 on the second and third pass when it fits).
template <typename T, bool BWD>
__global__ void __launch_bounds__(256) softmax_generic_kernel(const __grid_constant__ SmArgs a) {
  __shared__ float sm_a[8], sm_b[8];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int64_t row = blockIdx.x; row < a.rows; row += gridDim.x) {
    const T* p0 = static_cast<const T*>(a.in0) + row * a.cols;
    T* dst = static_cast<T*>(a.out) + row * a.cols;
    if (!BWD) {
      MS ms{-INFINITY, 0.0f};
      for (int64_t c = tid; c < a.cols; c += 256) {
        const float xv = to_f32<T>(p0[c]);
        ms = ms_merge(ms, MS{xv, xv == -INFINITY ? 0.0f : 1.0f});
      }
      ms = ms_shuffle_reduce<32>(ms);
      if (lane == 0) { sm_a[warp] = ms.m; sm_b[warp] = ms.s; }
      __syncthreads();
      MS acc{sm_a[0], sm_b[0]};
      for (int k = 1; k < 8; ++k) acc = ms_merge(acc, MS{sm_a[k], sm_b[k]});
      __syncthreads();
      for (int64_t c = tid; c < a.cols; c += 256) {
        const float xv = to_f32<T>(p0[c]);
        const float ev = (xv == -INFINITY && acc.m == -INFINITY) ? NAN : expf(xv - acc.m);
        dst[c] = from_f32<T>(__fdiv_rn(ev, acc.s));
      }
    } else {
      const T* p1 = static_cast<const T*>(a.in1) + row * a.cols;
      float d = 0.0f;
      for (int64_t c = tid; c < a.cols; c += 256) d = fmaf(to_f32<T>(p0[c]), to_f32<T>(p1[c]), d);
      d = warp_sum(d);
      if (lane == 0) sm_a[warp] = d;
      __syncthreads();
      float dot = 0.0f;
      for (int k = 0; k < 8; ++k) dot += sm_a[k];
      __syncthreads();
      for (int64_t c = tid; c < a.cols; c += 256)
        dst[c] = from_f32<T>((to_f32<T>(p0[c]) - dot) * to_f32<T>(p1[c]));
    }
  }
}

template <typename T, bool BWD, int TPR, int VPT>
int launch_cfg(const SmArgs& a, cudaStream_t s) {
  constexpr int NT = TPR > 256 ? TPR : 256;
  constexpr int RPC = NT / TPR;
  const int64_t grid = (a.rows + RPC - 1) / RPC;
  if (grid > 0x7fffffff) { set_error("softmax: too many rows for one launch"); return CDR_ERR_UNSUPPORTED; }
  if constexpr (BWD) softmax_bwd_kernel<T, TPR, VPT><<<static_cast<unsigned>(grid), NT, 0, s>>>(a);
  else softmax_fwd_kernel<T, TPR, VPT><<<static_cast<unsigned>(grid), NT, 0, s>>>(a);
  CDR_CUDA_TRY(cudaGetLastError());
  return CDR_OK;
}

template <typename T, bool BWD>
int launch_typed(const SmArgs& a, bool vec_ok, cudaStream_t s) {
  constexpr int V = Pack16<T>::N;
  const int64_t vec = a.cols / V;
  // at most 32 row elements per thread (they all stay in registers); the
  // 1024-thread backward variant holds two rows' worth and stops at 16
  constexpr int VMAX = 32 / V, VH = VMAX / 2;
  if (vec_ok) {
    if (vec <= 8) return launch_cfg<T, BWD, 8, 1>(a, s);
    if (vec <= 16) return launch_cfg<T, BWD, 16, 1>(a, s);
    if (vec <= 32) return launch_cfg<T, BWD, 32, 1>(a, s);
    if (vec <= 64) return launch_cfg<T, BWD, 32, 2>(a, s);
    if (vec <= 32 * VH) return launch_cfg<T, BWD, 32, VH>(a, s);
    if (vec <= 64 * VH) return launch_cfg<T, BWD, 64, VH>(a, s);
    if (vec <= 128 * VH) return launch_cfg<T, BWD, 128, VH>(a, s);
    if (vec <= 256 * VH) return launch_cfg<T, BWD, 256, VH>(a, s);
    if (vec <= 256 * VMAX) return launch_cfg<T, BWD, 256, VMAX>(a, s);
    if (vec <= 512 * VMAX) return launch_cfg<T, BWD, 512, VMAX>(a, s);
    if (vec <= 1024 * VH) return launch_cfg<T, BWD, 1024, VH>(a, s);
    if (!BWD && vec <= 1024 * VMAX) return launch_cfg<T, false, 1024, VMAX>(a, s);
  }
  int64_t grid = a.rows;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  if (grid > cap) grid = cap;
  softmax_generic_kernel<T, BWD><<<static_cast<unsigned>(grid), 256, 0, s>>>(a);
  CDR_CUDA_TRY(cudaGetLastError());
  return CDR_OK;
}

template <bool BWD>
int launch_softmax(const cdr_tensor* ins, int n_in, const cdr_tensor* outs, int n_out, cudaStream_t stream) {
  const char* who = BWD ? "softmax_bwd" : "softmax_fwd";
  const int want_in = BWD ? 2 : 1;
  if (n_in != want_in || n_out != 1 || !ins || !outs) {
    set_error("%s: expects %d input(s) and 1 output, got %d and %d", who, want_in, n_in, n_out);
    return CDR_ERR_BAD_ARG;
  }
  const cdr_tensor& x = ins[0];
  const cdr_tensor& out = outs[0];
  if (x.rank < 1) { set_error("%s: rank-0 input", who); return CDR_ERR_BAD_ARG; }
  const int64_t cols = x.shape[x.rank - 1];
  const int64_t n = numel(x);
  const int64_t rows = cols ? n / cols : 0;
  bool vec_ok = true;
  for (int i = 0; i < n_in; ++i) {
    if (ins[i].dtype != x.dtype || numel(ins[i]) != n || !is_contiguous(ins[i])) {
      set_error("%s: input %d must be contiguous, same dtype and element count as input 0", who, i);
      return CDR_ERR_BAD_ARG;
    }
    if (n && !ins[i].data) { set_error("%s: input %d has a null pointer", who, i); return CDR_ERR_BAD_ARG; }
    vec_ok &= aligned16(ins[i].data);
  }
  if (out.dtype != x.dtype || numel(out) != n || !is_contiguous(out)) {
    set_error("%s: output must be contiguous with the input's dtype and element count", who);
    return CDR_ERR_BAD_ARG;
  }
  if (n == 0) return CDR_OK;
  if (!out.data) { set_error("%s: output pointer is null", who); return CDR_ERR_BAD_ARG; }
  vec_ok &= aligned16(out.data);
  const int esz = dtype_size(x.dtype);
  if (x.dtype != CDR_F32 && x.dtype != CDR_BF16 && x.dtype != CDR_F16) {
    set_error("%s: dtype %d unsupported", who, x.dtype);
    return CDR_ERR_UNSUPPORTED;
  }
  vec_ok &= (cols % (16 / esz) == 0);
  SmArgs a{ins[0].data, BWD ? ins[1].data : nullptr, out.data, rows, cols};
  if (x.dtype == CDR_F32) return launch_typed<float, BWD>(a, vec_ok, stream);
  if (x.dtype == CDR_BF16) return launch_typed<__nv_bfloat16, BWD>(a, vec_ok, stream);
  return launch_typed<__half, BWD>(a, vec_ok, stream);
}

}  // namespace

int launch_softmax_fwd(const cdr_tensor* ins, int n_in, const cdr_tensor* outs, int n_out, cudaStream_t stream) {
  return launch_softmax<false>(ins, n_in, outs, n_out, stream);
}
int launch_softmax_bwd(const cdr_tensor* ins, int n_in, const cdr_tensor* outs, int n_out, cudaStream_t stream) {
  return launch_softmax<true>(ins, n_in, outs, n_out, stream);
}

}  // namespace cdr
