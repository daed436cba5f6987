// K5 -- fused scaled-dot-product attention:  O = softmax(Q K^T * scale [+ causal mask]) V.
//
// Reference definitions: the three-phase kernels of choreo-op/attention-gcu-only-test.co:15-134 and
// efficientattention-gcu-only-test.co:13-126, and the per-row online-softmax recurrence of
// choreo-op/flashattention-gcu-only-test.co:75-122 (d_i = d_prev*e^(m_prev-m) + e^(s-m)); the
// executed path is eager torch.nn.functional.scaled_dot_product_attention in bf16.
//
// Tensor-core bound.  One CTA per (batch*head, 128-query tile); key/value blocks of 128:
//   warp 0     TMA producer: Q once, then K_j and V_j into two-stage rings (128-byte swizzle)
//   warp 1     MMA issuer: S_j = Q K_j^T (tcgen05.mma, fp32 in TMEM, double buffered so that
//              S_{j+1} is computed while the softmax of block j runs) and O += P_j V_j
//   warps 2-5  softmax: one query row per thread; tcgen05.ld the S row, running max / sum in the
//              log2 domain, P_j = exp2(..) rounded to bf16 and written to shared memory in the
//              swizzled K-major layout the second MMA reads; the O accumulator stays in TMEM
//              and is rescaled (tcgen05.ld/st) only when the running max grew by more than 2^8,
//              which keeps P within bf16 range and is exact after the final division by the sum
// Causal work is triangular, so CTAs are numbered heaviest tile first.  No load is multicast;
// every wait is bounded and reports through the device status word.
#include <cuda.h>
#include <math.h>

#include "cdr_common.cuh"
#include "cdr_sm100.cuh"

namespace cdr {

int make_tensor_map_3d(CUtensorMap* map, const void* base, int is_bf16, int64_t d0, int64_t d1, int64_t d2,
                       int box0, int box1);

namespace {

constexpr int BQ = 128, BKV = 128;
constexpr int ATT_THREADS = 192;
constexpr int TMEM_S0 = 0, TMEM_S1 = 128, TMEM_O = 256, ATT_TMEM_COLS = 512;
constexpr float kRescaleThreshold = 8.0f;  // log2 units

struct AttnArgs {
  CUtensorMap tmap_q, tmap_k, tmap_v;  // [BH, S, D] each, box 64 x 128 x 1
  void* out;                            // [BH, S, D]
  int S, BH, n_qtiles;
  float scale_log2;                     // scale * log2(e)
  int causal;
  int* status;
};

template <int HD>
struct AttnSmem {
  static constexpr int TILE_BYTES = 128 * HD * 2;      // Q, K or V tile
  static constexpr int P_BYTES = BQ * BKV * 2;
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = TILE_BYTES;             // 2 stages
  static constexpr int V_OFF = K_OFF + 2 * TILE_BYTES; // 2 stages
  static constexpr int P_OFF = V_OFF + 2 * TILE_BYTES;
  static constexpr int BAR_OFF = P_OFF + P_BYTES;
  static constexpr size_t TOTAL = BAR_OFF + 256 + 1024;
};

// barrier indices inside the barrier block
enum { B_QFULL = 0, B_KFULL = 1, B_KEMPTY = 3, B_VFULL = 5, B_VEMPTY = 7, B_SFULL = 9, B_SEMPTY = 11, B_PFULL = 13,
       B_PVDONE = 14, B_COUNT = 15 };

template <int HD, bool BF16>
__global__ void __launch_bounds__(ATT_THREADS, 1) attention_kernel(const __grid_constant__ AttnArgs a) {
  using L = AttnSmem<HD>;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + B_COUNT);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // heaviest (last) query tiles first
  const int q_tile = a.n_qtiles - 1 - static_cast<int>(blockIdx.x) / a.BH;
  const int bh = static_cast<int>(blockIdx.x) % a.BH;
  const int q0 = q_tile * BQ;
  const int kv_total = (a.S + BKV - 1) / BKV;
  int n_blocks = kv_total;
  if (a.causal) {
    const int lim = (q0 + BQ + BKV - 1) / BKV;
    n_blocks = lim < kv_total ? lim : kv_total;
  }

  if (warp == 0 && lane == 0) {
    sm100::prefetch_tensormap(&a.tmap_q);
    sm100::prefetch_tensormap(&a.tmap_k);
    sm100::prefetch_tensormap(&a.tmap_v);
    for (int i = 0; i < B_COUNT; ++i) {
      const bool four = (i == B_SEMPTY || i == B_SEMPTY + 1 || i == B_PFULL);  // one arrival per softmax warp
      sm100::mbar_init(&bars[i], four ? 4 : 1);
    }
    sm100::fence_barrier_init();
  }
  if (warp == 1) {
    sm100::tmem_alloc(tmem_slot, ATT_TMEM_COLS);
    sm100::tmem_relinquish();
  }
  sm100::tc_fence_before();
  __syncthreads();
  sm100::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      sm100::mbar_arrive_expect_tx(&bars[B_QFULL], L::TILE_BYTES);
#pragma unroll
      for (int h = 0; h < HD / 64; ++h)
        sm100::tma_load_3d(smem + L::Q_OFF + h * (128 * 128), &a.tmap_q, h * 64, q0, bh, &bars[B_QFULL]);
      for (int j = 0; j < n_blocks; ++j) {
        const int st = j & 1, use = j >> 1;
        if (use > 0 && !sm100::mbar_wait(&bars[B_KEMPTY + st], (use - 1) & 1)) { sm100::report_timeout(a.status, 20); break; }
        sm100::mbar_arrive_expect_tx(&bars[B_KFULL + st], L::TILE_BYTES);
#pragma unroll
        for (int h = 0; h < HD / 64; ++h)
          sm100::tma_load_3d(smem + L::K_OFF + st * L::TILE_BYTES + h * (128 * 128), &a.tmap_k, h * 64, j * BKV, bh,
                             &bars[B_KFULL + st]);
        if (use > 0 && !sm100::mbar_wait(&bars[B_VEMPTY + st], (use - 1) & 1)) { sm100::report_timeout(a.status, 21); break; }
        sm100::mbar_arrive_expect_tx(&bars[B_VFULL + st], L::TILE_BYTES);
#pragma unroll
        for (int h = 0; h < HD / 64; ++h)
          sm100::tma_load_3d(smem + L::V_OFF + st * L::TILE_BYTES + h * (128 * 128), &a.tmap_v, h * 64, j * BKV, bh,
                             &bars[B_VFULL + st]);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = sm100::umma_idesc_f16(BQ, BKV, BF16, false, false);
      constexpr uint32_t idesc_o = sm100::umma_idesc_f16(BQ, HD, BF16, false, true);  // V is MN-major
      const uint32_t q_addr = sm100::smem_u32(smem + L::Q_OFF);
      const uint32_t p_addr = sm100::smem_u32(smem + L::P_OFF);
      bool ok = sm100::mbar_wait(&bars[B_QFULL], 0);
      if (!ok) sm100::report_timeout(a.status, 22);

      auto issue_s = [&](int j) -> bool {
        const int st = j & 1, use = j >> 1;
        if (!sm100::mbar_wait(&bars[B_KFULL + st], use & 1)) { sm100::report_timeout(a.status, 23); return false; }
        if (use > 0 && !sm100::mbar_wait(&bars[B_SEMPTY + st], (use - 1) & 1)) { sm100::report_timeout(a.status, 24); return false; }
        sm100::tc_fence_after();
        const uint32_t k_addr = sm100::smem_u32(smem + L::K_OFF + st * L::TILE_BYTES);
        const uint32_t d = tmem_base + (st ? TMEM_S1 : TMEM_S0);
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = (kk / 4) * (128 * 128) + (kk % 4) * 32;
          sm100::umma_f16_ss(d, sm100::umma_desc_k_sw128(q_addr + off), sm100::umma_desc_k_sw128(k_addr + off), idesc_s,
                             kk > 0 ? 1u : 0u);
        }
        sm100::umma_commit(&bars[B_KEMPTY + st]);
        sm100::umma_commit(&bars[B_SFULL + st]);
        return true;
      };

      if (ok) ok = issue_s(0);
      for (int j = 0; j < n_blocks && ok; ++j) {
        if (j + 1 < n_blocks) { ok = issue_s(j + 1); if (!ok) break; }
        const int st = j & 1, use = j >> 1;
        if (!sm100::mbar_wait(&bars[B_VFULL + st], use & 1)) { sm100::report_timeout(a.status, 25); break; }
        if (!sm100::mbar_wait(&bars[B_PFULL], j & 1)) { sm100::report_timeout(a.status, 26); break; }
        sm100::tc_fence_after();
        const uint32_t v_addr = sm100::smem_u32(smem + L::V_OFF + st * L::TILE_BYTES);
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk) {
          const uint32_t p_off = (kk / 4) * (128 * 128) + (kk % 4) * 32;
          const uint64_t pdesc = sm100::umma_desc_k_sw128(p_addr + p_off);
          const uint64_t vdesc = sm100::umma_desc_mn_sw128(v_addr + kk * (16 * 128), 128 * 128);
          sm100::umma_f16_ss(tmem_base + TMEM_O, pdesc, vdesc, idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
        }
        sm100::umma_commit(&bars[B_VEMPTY + st]);
        sm100::umma_commit(&bars[B_PVDONE]);
      }
    }
  } else {
    // ------------------------------------------------------------ softmax / correction / epilogue
    const int q = warp & 3;
    const int row_in_tile = q * 32 + lane;
    const int row = q0 + row_in_tile;
    const uint32_t lane_sel = static_cast<uint32_t>(q * 32) << 16;
    unsigned char* p_smem = smem + L::P_OFF;
    float m_ref = -INFINITY, l_sum = 0.0f;
    bool ok = true;

    for (int j = 0; j < n_blocks; ++j) {
      const int st = j & 1, use = j >> 1;
      if (!sm100::mbar_wait(&bars[B_SFULL + st], use & 1)) { sm100::report_timeout(a.status, 27); ok = false; break; }
      sm100::tc_fence_after();
      uint32_t sr[4][32];
      const uint32_t s_addr = tmem_base + (st ? TMEM_S1 : TMEM_S0) + lane_sel;
#pragma unroll
      for (int c = 0; c < 4; ++c) sm100::tmem_ld32(s_addr + c * 32, sr[c]);
      sm100::tmem_ld_wait();
      sm100::tc_fence_before();
      __syncwarp();
      if (lane == 0) sm100::mbar_arrive(&bars[B_SEMPTY + st]);  // this S buffer may be overwritten

      const int key0 = j * BKV;
      const bool need_mask = (a.causal && key0 + BKV - 1 > q0) || (key0 + BKV > a.S);
      float bmax = -INFINITY;
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float v = __uint_as_float(sr[c][i]);
          if (need_mask) {
            const int key = key0 + c * 32 + i;
            if (key >= a.S || (a.causal && key > row)) v = -INFINITY;
            sr[c][i] = __float_as_uint(v);
          }
          bmax = fmaxf(bmax, v);
        }
      bmax *= a.scale_log2;  // scale > 0: max commutes with the scaling

      // block j-1's P V must be complete before O is touched or the P buffer rewritten
      if (j > 0 && !sm100::mbar_wait(&bars[B_PVDONE], (j - 1) & 1)) { sm100::report_timeout(a.status, 28); ok = false; break; }
      sm100::tc_fence_after();

      if (j == 0) {
        m_ref = bmax;
      } else if (__any_sync(0xffffffffu, bmax > m_ref + kRescaleThreshold)) {
        const float m_new = fmaxf(m_ref, bmax);
        const float alpha = (m_ref == -INFINITY) ? 0.0f : exp2f(m_ref - m_new);
        l_sum *= alpha;
        m_ref = m_new;
#pragma unroll 1
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t o[32];
          sm100::tmem_ld32(tmem_base + TMEM_O + lane_sel + c * 32, o);
          sm100::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          sm100::tmem_st32(tmem_base + TMEM_O + lane_sel + c * 32, o);
        }
        sm100::tmem_st_wait();
      }

      // P = exp2(s*c - m), bf16, written as the K-major swizzled A operand of the second MMA
      const float neg_m = (m_ref == -INFINITY) ? 0.0f : -m_ref;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint32_t w[4];
#pragma unroll
          for (int h = 0; h < 4; ++h) {
            const float p0 = exp2f(fmaf(__uint_as_float(sr[c][g * 8 + h * 2]), a.scale_log2, neg_m));
            const float p1 = exp2f(fmaf(__uint_as_float(sr[c][g * 8 + h * 2 + 1]), a.scale_log2, neg_m));
            l_sum += p0 + p1;
            if (BF16) { __nv_bfloat162 t = __floats2bfloat162_rn(p0, p1); w[h] = *reinterpret_cast<uint32_t*>(&t); }
            else { __half2 t = __floats2half2_rn(p0, p1); w[h] = *reinterpret_cast<uint32_t*>(&t); }
          }
          const int key = c * 32 + g * 8;                 // first of 8 keys in this 16-byte chunk
          const int half = key >> 6, chunk = (key & 63) >> 3;
          unsigned char* dst = p_smem + half * (128 * 128) + row_in_tile * 128 + ((chunk ^ (row_in_tile & 7)) << 4);
          *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
      sm100::fence_proxy_async_smem();   // generic-proxy writes of P -> visible to the MMA (async proxy)
      sm100::tc_fence_before();
      __syncwarp();
      if (lane == 0) sm100::mbar_arrive(&bars[B_PFULL]);
    }

    // ---- epilogue: O / l, rounded to the output type
    if (ok && n_blocks > 0) {
      if (!sm100::mbar_wait(&bars[B_PVDONE], (n_blocks - 1) & 1)) { sm100::report_timeout(a.status, 29); ok = false; }
    }
    if (ok) {
      sm100::tc_fence_after();
      const float inv = 1.0f / l_sum;
      unsigned char* orow = static_cast<unsigned char*>(a.out) + (static_cast<size_t>(bh) * a.S + row) * (HD * 2);
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t o[32];
        sm100::tmem_ld32(tmem_base + TMEM_O + lane_sel + c * 32, o);
        sm100::tmem_ld_wait();
        if (row < a.S) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint32_t w[4];
#pragma unroll
            for (int h = 0; h < 4; ++h) {
              const float x0 = __uint_as_float(o[g * 8 + h * 2]) * inv, x1 = __uint_as_float(o[g * 8 + h * 2 + 1]) * inv;
              if (BF16) { __nv_bfloat162 t = __floats2bfloat162_rn(x0, x1); w[h] = *reinterpret_cast<uint32_t*>(&t); }
              else { __half2 t = __floats2half2_rn(x0, x1); w[h] = *reinterpret_cast<uint32_t*>(&t); }
            }
            *reinterpret_cast<uint4*>(orow + c * 64 + g * 16) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
    }
  }

  sm100::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    sm100::tc_fence_after();
    sm100::tmem_dealloc(tmem_base, ATT_TMEM_COLS);
  }
}

}  // namespace

// ---------------------------------------------------------------- host side
int attention_workspace(const cdr_tensor*, int, size_t* bytes) {
  *bytes = 0;  // O, the running max and the running sum never leave TMEM / registers
  return CDR_OK;
}

namespace {
template <int HD, bool BF16>
int launch_attention_cfg(const AttnArgs& a, cudaStream_t stream) {
  auto kern = attention_kernel<HD, BF16>;
  constexpr size_t smem = AttnSmem<HD>::TOTAL;
  static bool configured_dev[64] = {false};
  int dev = 0;
  CDR_CUDA_TRY(cudaGetDevice(&dev));
  if (!configured_dev[dev & 63]) {
    CDR_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    configured_dev[dev & 63] = true;
  }
  const int64_t grid = static_cast<int64_t>(a.BH) * a.n_qtiles;
  if (grid > 0x7fffffff) { set_error("attention: too many tiles"); return CDR_ERR_UNSUPPORTED; }
  kern<<<static_cast<unsigned>(grid), ATT_THREADS, smem, stream>>>(a);
  CDR_CUDA_TRY(cudaGetLastError());
  return CDR_OK;
}
}  // namespace

int launch_attention(const cdr_tensor* ins, int n_in, const cdr_tensor* outs, int n_out, const cdr_attn_params* p,
                     void*, size_t, cudaStream_t stream) {
  if (!p) { set_error("attention: params is null"); return CDR_ERR_BAD_ARG; }
  if (n_in != 3 || n_out != 1) { set_error("attention: expects (q, k, v) and one output"); return CDR_ERR_BAD_ARG; }
  const cdr_tensor& q = ins[0];
  if (q.rank < 2) { set_error("attention: q needs rank >= 2"); return CDR_ERR_BAD_ARG; }
  const int64_t D = q.shape[q.rank - 1], S = q.shape[q.rank - 2];
  const int64_t n = numel(q);
  const int64_t BH = (S * D) ? n / (S * D) : 0;
  for (int i = 0; i < 3; ++i) {
    if (ins[i].rank != q.rank || ins[i].dtype != q.dtype || !is_contiguous(ins[i])) {
      set_error("attention: q, k, v must be contiguous with one rank and dtype");
      return CDR_ERR_BAD_ARG;
    }
    for (int d = 0; d < q.rank; ++d)
      if (ins[i].shape[d] != q.shape[d]) {
        set_error("attention: q, k, v must have identical shapes (no cross-attention lengths, no grouped heads)");
        return CDR_ERR_UNSUPPORTED;
      }
  }
  const cdr_tensor& out = outs[0];
  if (out.dtype != q.dtype || numel(out) != n || !is_contiguous(out)) {
    set_error("attention: output must match q in dtype and element count");
    return CDR_ERR_BAD_ARG;
  }
  if (q.dtype != CDR_BF16 && q.dtype != CDR_F16) { set_error("attention: dtype %d unsupported (bf16 and f16 only)", q.dtype); return CDR_ERR_UNSUPPORTED; }
  if (D != 64 && D != 128) { set_error("attention: head dim %lld unsupported (64 or 128)", (long long)D); return CDR_ERR_UNSUPPORTED; }
  if (!(p->scale > 0.0f) || !isfinite(p->scale)) { set_error("attention: scale must be positive and finite"); return CDR_ERR_UNSUPPORTED; }
  if (n == 0) return CDR_OK;
  for (int i = 0; i < 3; ++i)
    if (!ins[i].data || !aligned16(ins[i].data)) { set_error("attention: input %d is null or not 16-byte aligned", i); return CDR_ERR_MISALIGNED; }
  if (!out.data || !aligned16(out.data)) { set_error("attention: output is null or not 16-byte aligned"); return CDR_ERR_MISALIGNED; }
  if (S > 0x7fffffff || BH > 0x7fffffff) { set_error("attention: extent too large"); return CDR_ERR_UNSUPPORTED; }

  AttnArgs a;
  const int bf16 = q.dtype == CDR_BF16;
  if (int rc = make_tensor_map_3d(&a.tmap_q, ins[0].data, bf16, D, S, BH, 64, 128)) return rc;
  if (int rc = make_tensor_map_3d(&a.tmap_k, ins[1].data, bf16, D, S, BH, 64, 128)) return rc;
  if (int rc = make_tensor_map_3d(&a.tmap_v, ins[2].data, bf16, D, S, BH, 64, 128)) return rc;
  a.out = out.data;
  a.S = static_cast<int>(S);
  a.BH = static_cast<int>(BH);
  a.n_qtiles = static_cast<int>((S + BQ - 1) / BQ);
  a.scale_log2 = p->scale * 1.4426950408889634f;
  a.causal = p->causal ? 1 : 0;
  a.status = device_status_ptr();
  if (D == 128) return bf16 ? launch_attention_cfg<128, true>(a, stream) : launch_attention_cfg<128, false>(a, stream);
  return bf16 ? launch_attention_cfg<64, true>(a, stream) : launch_attention_cfg<64, false>(a, stream);
}

}  // namespace cdr
