// K6 -- layer normalisation over the last dimension, one pass over memory.
//
// y = (x - mean(x)) / sqrt(var(x) + eps) * w + b with the biased variance, as
// torch.nn.functional.layer_norm computes it (statistics in fp32, one rounding to the output type).
// The reference has no kernel for it (its operator lists stop at elementwise ops and reductions,
// conductor/optimization/fusion.py:652-675); the skeleton is the row softmax's: a row is loaded
// once with 128-bit streaming loads and stays in registers until its result is stored, the two
// row statistics go through warp shuffles and one shared-memory hop each.  The variance is the
// mean of squared deviations from the mean (two passes over registers, not E[x^2] - E[x]^2).
// Rows that do not fit the register-resident variants (more than 32 elements per thread at 1024
// threads, or a ragged / misaligned row) are reported as unsupported; the caller then lowers
// layer_norm to two row reductions and an elementwise chain instead.
#include <math.h>

#include "cdr_common.cuh"

namespace cdr {
namespace {

struct LnArgs {
  const void* x;
  const void* w;   // [cols] or nullptr
  const void* b;   // [cols] or nullptr
  void* out;
  int64_t rows;
  int64_t cols;
  float eps;
};

template <int WIDTH>
__device__ __forceinline__ float ln_shuffle_sum(float v) {
#pragma unroll
  for (int o = WIDTH / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// TPR threads cooperate on one row; a CTA holds max(256, TPR) threads, i.e. 256/TPR rows.
template <typename T, int TPR, int VPT>
__global__ void __launch_bounds__((TPR > 256 ? TPR : 256)) layer_norm_kernel(const __grid_constant__ LnArgs a) {
  constexpr int V = Pack16<T>::N;
  constexpr int NT = TPR > 256 ? TPR : 256;
  constexpr int RPC = NT / TPR;                  // rows per CTA
  constexpr int WPR = TPR > 32 ? TPR / 32 : 1;   // warps per row
  __shared__ float sm_a[RPC][WPR], sm_b[RPC][WPR];

  const int tid = threadIdx.x;
  const int rloc = tid / TPR, t = tid % TPR;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * RPC + rloc;
  const bool live = row < a.rows;
  const int64_t vec_per_row = a.cols / V;
  const T* src = static_cast<const T*>(a.x) + (live ? row : 0) * a.cols;

  float x[VPT][V];
  float s = 0.0f;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int64_t v = t + static_cast<int64_t>(j) * TPR;
    if (live && v < vec_per_row) {
      Pack16<T>::unpack(ld_stream16(src + v * V), x[j]);
    } else {
#pragma unroll
      for (int e = 0; e < V; ++e) x[j][e] = 0.0f;
    }
#pragma unroll
    for (int e = 0; e < V; ++e) s += x[j][e];
  }
  auto row_sum = [&](float v, float (*sm)[WPR]) {
    v = ln_shuffle_sum<(TPR < 32 ? TPR : 32)>(v);
    if (WPR > 1) {
      const int w = t >> 5;
      if ((t & 31) == 0) sm[rloc][w] = v;
      __syncthreads();
      float acc = sm[rloc][0];
#pragma unroll
      for (int k = 1; k < WPR; ++k) acc += sm[rloc][k];
      v = acc;
    }
    return v;
  };
  const float inv_n = 1.0f / static_cast<float>(a.cols);
  const float mean = row_sum(s, sm_a) * inv_n;

  float q = 0.0f;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int64_t v = t + static_cast<int64_t>(j) * TPR;
    const bool in_row = live && v < vec_per_row;
#pragma unroll
    for (int e = 0; e < V; ++e) {
      const float d = in_row ? x[j][e] - mean : 0.0f;   // padding must not count as (0 - mean)^2
      x[j][e] = d;
      q += d * d;
    }
  }
  const float var = row_sum(q, sm_b) * inv_n;
  const float rstd = __fdiv_rn(1.0f, __fsqrt_rn(var + a.eps));

  T* dst = static_cast<T*>(a.out) + (live ? row : 0) * a.cols;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int64_t v = t + static_cast<int64_t>(j) * TPR;
    if (live && v < vec_per_row) {
      float y[V], wv[V], bv[V];
      if (a.w) Pack16<T>::unpack(ld_cached16(static_cast<const T*>(a.w) + v * V), wv);
      if (a.b) Pack16<T>::unpack(ld_cached16(static_cast<const T*>(a.b) + v * V), bv);
#pragma unroll
      for (int e = 0; e < V; ++e) {
        float r = x[j][e] * rstd;
        if (a.w) r *= wv[e];
        if (a.b) r += bv[e];
        y[e] = r;
      }
      st_stream16(dst + v * V, Pack16<T>::pack(y));
    }
  }
}

template <typename T, int TPR, int VPT>
int launch_cfg(const LnArgs& a, cudaStream_t s) {
  constexpr int NT = TPR > 256 ? TPR : 256;
  constexpr int RPC = NT / TPR;
  const int64_t grid = (a.rows + RPC - 1) / RPC;
  if (grid > 0x7fffffff) { set_error("layer_norm: too many rows for one launch"); return CDR_ERR_UNSUPPORTED; }
  layer_norm_kernel<T, TPR, VPT><<<static_cast<unsigned>(grid), NT, 0, s>>>(a);
  CDR_CUDA_TRY(cudaGetLastError());
  return CDR_OK;
}

template <typename T>
int launch_typed(const LnArgs& a, cudaStream_t s) {
  constexpr int V = Pack16<T>::N;
  const int64_t vec = a.cols / V;
  constexpr int VMAX = 32 / V, VH = VMAX / 2;   // at most 32 row elements per thread
  if (vec <= 8) return launch_cfg<T, 8, 1>(a, s);
  if (vec <= 16) return launch_cfg<T, 16, 1>(a, s);
  if (vec <= 32) return launch_cfg<T, 32, 1>(a, s);
  if (vec <= 64) return launch_cfg<T, 32, 2>(a, s);
  if (vec <= 32 * VH) return launch_cfg<T, 32, VH>(a, s);
  if (vec <= 64 * VH) return launch_cfg<T, 64, VH>(a, s);
  if (vec <= 128 * VH) return launch_cfg<T, 128, VH>(a, s);
  if (vec <= 256 * VH) return launch_cfg<T, 256, VH>(a, s);
  if (vec <= 256 * VMAX) return launch_cfg<T, 256, VMAX>(a, s);
  if (vec <= 512 * VMAX) return launch_cfg<T, 512, VMAX>(a, s);
  if (vec <= 1024 * VH) return launch_cfg<T, 1024, VH>(a, s);
  set_error("layer_norm: rows of %lld elements do not fit the register-resident kernel", (long long)a.cols);
  return CDR_ERR_UNSUPPORTED;
}

}  // namespace

int launch_layer_norm(const cdr_tensor* ins, int n_in, const cdr_tensor* outs, int n_out, const cdr_norm_params* p,
                      cudaStream_t stream) {
  if (!p) { set_error("layer_norm: params is null"); return CDR_ERR_BAD_ARG; }
  const int want_in = 1 + (p->has_weight ? 1 : 0) + (p->has_bias ? 1 : 0);
  if (n_in != want_in || n_out != 1 || !ins || !outs) {
    set_error("layer_norm: expects %d input(s) and 1 output, got %d and %d", want_in, n_in, n_out);
    return CDR_ERR_BAD_ARG;
  }
  const cdr_tensor& x = ins[0];
  const cdr_tensor& out = outs[0];
  if (x.rank < 1) { set_error("layer_norm: rank-0 input"); return CDR_ERR_BAD_ARG; }
  const int64_t cols = x.shape[x.rank - 1];
  const int64_t n = numel(x);
  const int64_t rows = cols ? n / cols : 0;
  if (x.dtype != CDR_F32 && x.dtype != CDR_BF16 && x.dtype != CDR_F16) {
    set_error("layer_norm: dtype %d unsupported", x.dtype);
    return CDR_ERR_UNSUPPORTED;
  }
  if (!is_contiguous(x) || out.dtype != x.dtype || numel(out) != n || !is_contiguous(out)) {
    set_error("layer_norm: input and output must be contiguous with one dtype and element count");
    return CDR_ERR_BAD_ARG;
  }
  if (!(p->eps >= 0.0f) || !isfinite(p->eps)) { set_error("layer_norm: eps must be finite and non-negative"); return CDR_ERR_BAD_ARG; }
  const int esz = dtype_size(x.dtype);
  bool vec_ok = aligned16(x.data) && aligned16(out.data) && cols % (16 / esz) == 0;
  for (int i = 1; i < n_in; ++i) {
    if (ins[i].dtype != x.dtype || numel(ins[i]) != cols || !is_contiguous(ins[i])) {
      set_error("layer_norm: weight / bias must hold %lld elements of the input's dtype", (long long)cols);
      return CDR_ERR_BAD_ARG;
    }
    if (n && !ins[i].data) { set_error("layer_norm: input %d has a null pointer", i); return CDR_ERR_BAD_ARG; }
    vec_ok &= aligned16(ins[i].data);
  }
  if (n == 0) return CDR_OK;
  if (!x.data || !out.data) { set_error("layer_norm: null pointer"); return CDR_ERR_BAD_ARG; }
  if (!vec_ok) { set_error("layer_norm: rows must be 16-byte aligned whole vectors"); return CDR_ERR_UNSUPPORTED; }
  LnArgs a{x.data, p->has_weight ? ins[1].data : nullptr, p->has_bias ? ins[1 + (p->has_weight ? 1 : 0)].data : nullptr,
           out.data, rows, cols, p->eps};
  if (x.dtype == CDR_F32) return launch_typed<float>(a, stream);
  if (x.dtype == CDR_BF16) return launch_typed<__nv_bfloat16>(a, stream);
  return launch_typed<__half>(a, stream);
}

}  // namespace cdr
