// K4 -- GEMM with fused bias + activation epilogue:  out[M,N] = act(x[M,K] @ W[N,K]^T + bias[N]).
//
// Reference definitions: the naive triple loop of choreo-op/matmul-gcu-only-test.co:8-16 and the
// string kernel conductor/codegen/device_kernels.py:84-103; the executed path is eager
// torch.nn.functional.linear (+ relu) in bf16 with fp32 accumulation.
//
// Tensor-core bound.  Blackwell-native structure, one persistent CTA per SM:
//   warp 0     TMA producer: 128x64 tile of x and 256x64 tile of W per k-block into a 4-stage
//              shared-memory ring (128-byte swizzle; both operands are K-major as stored)
//   warp 1     MMA issuer: one thread issues tcgen05.mma (M=128, N=256, K=16) x4 per k-block,
//              accumulating in tensor memory; tcgen05.commit releases the ring stage
//   warps 2-9  epilogue (two per TMEM lane quadrant, 128 columns each): tcgen05.ld the fp32 accumulator (lane = output row), add bias, ReLU,
//              round to bf16, store
// The accumulator is double buffered in TMEM (2 x 256 columns), so the epilogue of tile i runs
// under the MMAs of tile i+1.  Tiles are walked M-fastest so that concurrently running CTAs
// share the same weight tile in L2.  No load is multicast; every mbarrier wait is bounded.
// Measured and dropped: stream-K scheduling of the CTA-pair kernel for shapes whose last wave of
// tiles is badly filled (C4's second layer: 128 tiles on 74 pairs) -- equal shares of the
// (tile, k-block) sequence per pair, split tiles completed through fp32 partial tiles in scratch.
// It made the two-layer step 8 % slower (130 against 120 us): the pairs no longer walk the
// k-blocks of a shared weight tile in step, and the partial tiles add an L2 round trip to the
// epilogue.  Programmatic dependent launch between the two layers is in place and is neutral.
// Sixteen epilogue warps (four per TMEM lane quadrant) instead of eight: the K=1024 layer, whose
// epilogue per tile (8.4k cycles by clock64) is as long as its 16 k-blocks of MMAs and stalls the
// MMA warp for 12 % of the time, went 55-61 -> 63-64 us (96 registers per thread at 576 threads
// spill the double-buffered accumulator chunks).  Epilogue stores transposed through shared memory so
// that a warp writes four whole 128-byte lines per instruction instead of 32 sectors of 32 lines:
// no change (58-59 -> 60-62 us on the same box), so the scattered stores are not what holds it.
#include <cuda.h>

#include <cstdlib>

#include "cdr_common.cuh"
#include "cdr_sm100.cuh"

namespace cdr {
namespace {

constexpr int BM = 128, BN = 256, BK = 64, UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2;
constexpr int ACC_STAGES = 2;
constexpr int TMEM_COLS = ACC_STAGES * BN;  // 512: all of tensor memory
constexpr int NUM_THREADS = 320;          // TMA warp, MMA warp, 8 epilogue warps
constexpr int EPI_WARPS = 8;              // two per TMEM lane quadrant, half of the accumulator columns each
constexpr int EPI_CHUNKS = BN / 32 / 2;   // 32-column chunks per epilogue warp (256-column tiles)

// Geometry of the 1-CTA kernel for a tile of 128 x TN outputs.  TN = 256 is the default; TN = 128
// serves problems with so few 256-wide tiles that most SMs would idle (a 1024 x 1024 output is 16
// CTA-pair tiles on 74 pairs, but 64 tiles of 128 x 128).
template <int TN>
struct Tile1 {
  static constexpr int B_BYTES = TN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = TN == 256 ? 4 : 6;
  static constexpr int TMEM = ACC_STAGES * TN;
  static constexpr int CHUNKS = TN / 32 / 2;
  static constexpr size_t SMEM = static_cast<size_t>(STAGES) * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

struct GemmArgs {
  CUtensorMap tmap_a;  // x  [M, K], box 64 x 128 -- or, with x_km, x [K, M], box 64 (M) x 64 (K)
  CUtensorMap tmap_b;  // W  [N, K], box 64 x 256 -- or, with w_kn, W [K, N], box 64 (N) x 64 (K)
  const void* bias;    // [N] or nullptr
  const void* gate;    // [M, N] or nullptr: entries <= 0 (or NaN) zero the result at their position
  void* out;           // [M, N]
  int M, N, K;
  int relu;
  int is_bf16;
  int w_kn;            // W is stored [K, N] (N contiguous): the B operand is MN-major
  int x_km;            // x is stored [K, M] (M contiguous): the A operand is MN-major
  int tiles_m, tiles_n;
  int* status;
};

template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  if (BF16) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
// 256-bit global store (sm_100): p must be 32-byte aligned
__device__ __forceinline__ void st_global_v8(void* p, const uint32_t* w) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(w[0]), "r"(w[1]), "r"(w[2]),
               "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
               : "memory");
}

template <bool BF16>
__device__ __forceinline__ float load_elem(const void* p, int i) {
  if (BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
  return __half2float(static_cast<const __half*>(p)[i]);
}
template <bool BF16>
__device__ __forceinline__ void store_elem(void* p, size_t i, float v) {
  if (BF16) static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
  else static_cast<__half*>(p)[i] = __float2half_rn(v);
}

// Epilogue of one 128 x 256 accumulator tile for the thread that owns `row`: TMEM -> registers in
// 32-column chunks (the load of chunk c+1 is in flight while chunk c is processed), + bias,
// round to the output type, ReLU on the packed pairs (NaN-propagating max), 16-byte stores.
// Bias values are fetched with warp-uniform 128-bit loads issued before the TMEM wait.
template <bool BF16, int CHUNKS = EPI_CHUNKS>
__device__ __forceinline__ void epilogue_tile(const GemmArgs& a, uint32_t t_base, int row, int n0, bool vec_ok,
                                              int c_begin) {
  uint32_t r[2][32];
  sm100::tmem_ld32(t_base + c_begin * 32, r[0]);
  const bool bias_vec = a.bias != nullptr && vec_ok && (reinterpret_cast<uintptr_t>(a.bias) & 15u) == 0;
  if (a.gate != nullptr && (reinterpret_cast<uintptr_t>(a.gate) & 15u) != 0) vec_ok = false;   // the scalar path reads the gate element-wise
#pragma unroll
  for (int cc = 0; cc < CHUNKS; ++cc) {
    const int c = c_begin + cc;
    const int col0 = n0 + c * 32;
    const bool full_chunk = vec_ok && col0 + 32 <= a.N;
    uint4 bq[4] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
    uint4 gq[4];
    const bool gated = a.gate != nullptr;
    if (gated && full_chunk && row < a.M) {      // 64 bytes of this thread's row of the gate tensor
      const uint4* gp = reinterpret_cast<const uint4*>(static_cast<const unsigned char*>(a.gate) +
                                                       (static_cast<size_t>(row) * a.N + col0) * 2);
#pragma unroll
      for (int g = 0; g < 4; ++g) gq[g] = __ldg(gp + g);
    }
    if (bias_vec && full_chunk) {
      const uint4* bp = reinterpret_cast<const uint4*>(static_cast<const unsigned char*>(a.bias) + static_cast<size_t>(col0) * 2);
#pragma unroll
      for (int g = 0; g < 4; ++g) bq[g] = __ldg(bp + g);
    }
    sm100::tmem_ld_wait();
    if (cc + 1 < CHUNKS) sm100::tmem_ld32(t_base + (c + 1) * 32, r[(cc + 1) & 1]);
    const uint32_t* rc = r[cc & 1];
    if (row < a.M && col0 < a.N) {
      const size_t off = static_cast<size_t>(row) * a.N + col0;
      if (full_chunk && (bias_vec || a.bias == nullptr)) {
        unsigned char* dst = static_cast<unsigned char*>(a.out) + off * 2;
        const bool wide = ((a.N & 15) == 0) && ((reinterpret_cast<uintptr_t>(a.out) & 31u) == 0);  // 32-byte aligned rows
        uint32_t w[16];
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const uint32_t bw[4] = {bq[g].x, bq[g].y, bq[g].z, bq[g].w};
#pragma unroll
          for (int h = 0; h < 4; ++h) {
            float b0, b1;
            if (BF16) { b0 = __uint_as_float(bw[h] << 16); b1 = __uint_as_float(bw[h] & 0xffff0000u); }
            else { const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&bw[h])); b0 = f.x; b1 = f.y; }
            uint32_t v = pack2<BF16>(__uint_as_float(rc[g * 8 + h * 2]) + b0, __uint_as_float(rc[g * 8 + h * 2 + 1]) + b1);
            if (a.relu) {
              if (BF16) {
                const __nv_bfloat162 z = __float2bfloat162_rn(0.0f);
                __nv_bfloat162 t = __hmax2_nan(*reinterpret_cast<__nv_bfloat162*>(&v), z);
                v = *reinterpret_cast<uint32_t*>(&t);
              } else {
                const __half2 z = __float2half2_rn(0.0f);
                __half2 t = __hmax2_nan(*reinterpret_cast<__half2*>(&v), z);
                v = *reinterpret_cast<uint32_t*>(&t);
              }
            }
            if (gated) {
              // both 16-bit floats are sign + magnitude: positive means sign clear and magnitude non-zero (NaN counts
              // as not positive, as in `H > 0`)
              const uint32_t gw = (&gq[g].x)[h];
              const uint32_t lo = (gw & 0x8000u) == 0 && (gw & 0x7fffu) != 0 && (gw & 0x7fffu) <= (BF16 ? 0x7f80u : 0x7c00u) ? 0x0000ffffu : 0u;
              const uint32_t hw = gw >> 16;
              const uint32_t hi = (hw & 0x8000u) == 0 && (hw & 0x7fffu) != 0 && (hw & 0x7fffu) <= (BF16 ? 0x7f80u : 0x7c00u) ? 0xffff0000u : 0u;
              v &= lo | hi;
            }
            w[g * 4 + h] = v;
          }
        }
        if (wide) {   // two 256-bit stores: every store fills a whole 32-byte sector
          st_global_v8(dst, w);
          st_global_v8(dst + 32, w + 8);
        } else {
#pragma unroll
          for (int g = 0; g < 4; ++g)
            reinterpret_cast<uint4*>(dst)[g] = make_uint4(w[g * 4], w[g * 4 + 1], w[g * 4 + 2], w[g * 4 + 3]);
        }
      } else {
        for (int j = 0; j < 32 && col0 + j < a.N; ++j) {
          float x = __uint_as_float(rc[j]);
          if (a.bias != nullptr) x += load_elem<BF16>(a.bias, col0 + j);
          if (a.relu) x = x > 0.0f ? x : (x != x ? x : 0.0f);
          if (gated) {
            const float gv = BF16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(a.gate)[off + j])
                                  : __half2float(static_cast<const __half*>(a.gate)[off + j]);
            if (!(gv > 0.0f)) x = 0.0f;
          }
          store_elem<BF16>(a.out, off + j, x);
        }
      }
    }
  }
}

template <bool BF16, int TN>
__global__ void __launch_bounds__(NUM_THREADS, 1) gemm_epilogue_kernel(const __grid_constant__ GemmArgs a) {
  using G = Tile1<TN>;
  constexpr int STAGES = G::STAGES, STAGE_BYTES = G::STAGE_BYTES;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;
  uint64_t* acc_empty = acc_full + ACC_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + ACC_STAGES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp == 0 && lane == 0) {
    sm100::prefetch_tensormap(&a.tmap_a);
    sm100::prefetch_tensormap(&a.tmap_b);
    for (int s = 0; s < STAGES; ++s) {
      sm100::mbar_init(&full[s], 1);
      sm100::mbar_init(&empty[s], 1);
    }
    for (int s = 0; s < ACC_STAGES; ++s) {
      sm100::mbar_init(&acc_full[s], 1);
      sm100::mbar_init(&acc_empty[s], EPI_WARPS);  // one arrival per epilogue warp
    }
    sm100::fence_barrier_init();
  }
  if (warp == 1) {
    sm100::tmem_alloc(tmem_slot, G::TMEM);
    sm100::tmem_relinquish();
  }
  sm100::tc_fence_before();
  __syncthreads();
  sm100::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Programmatic dependent launch: everything above (barriers, tensor memory, descriptor prefetch)
  // may run while the previous kernel in the stream drains; nothing below touches global memory
  // before that kernel has completed and flushed.  No-ops without the launch attribute.
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");

  const int num_tiles = a.tiles_m * a.tiles_n;
  const int kblocks = (a.K + BK - 1) / BK;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile % a.tiles_m) * BM, n0 = (tile / a.tiles_m) * TN;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
          if (!sm100::mbar_wait(&empty[s], ph ^ 1)) { sm100::report_timeout(a.status, 10); ok = false; break; }
          sm100::mbar_arrive_expect_tx(&full[s], STAGE_BYTES);
          unsigned char* st = smem + s * STAGE_BYTES;
          if (!a.x_km) {
            sm100::tma_load_2d(st, &a.tmap_a, kb * BK, m0, &full[s]);
          } else {   // [K, M]: one box of 64 k-rows per 64 rows of the tile
#pragma unroll
            for (int c = 0; c < BM / 64; ++c)
              sm100::tma_load_2d(st + c * (BK * 128), &a.tmap_a, m0 + c * 64, kb * BK, &full[s]);
          }
          if (!a.w_kn) {
            sm100::tma_load_2d(st + A_BYTES, &a.tmap_b, kb * BK, n0, &full[s]);
          } else {   // [K, N]: one box of 64 k-rows per 64 columns of N
#pragma unroll
            for (int c = 0; c < TN / 64; ++c)
              sm100::tma_load_2d(st + A_BYTES + c * (BK * 128), &a.tmap_b, n0 + c * 64, kb * BK, &full[s]);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    // The whole warp runs the loop convergently and one elected lane issues the tcgen05
    // instructions, so the operand descriptors stay in uniform registers.
    {
      const bool leader = sm100::elect_one();
      const uint32_t idesc = sm100::umma_idesc_f16(BM, TN, BF16, a.x_km != 0, a.w_kn != 0);
      uint32_t it = 0, tile_iter = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tile_iter) {
        const uint32_t as = tile_iter % ACC_STAGES, aph = (tile_iter / ACC_STAGES) & 1;
        if (!__all_sync(0xffffffffu, sm100::mbar_wait(&acc_empty[as], aph ^ 1))) {
          if (leader) sm100::report_timeout(a.status, 11);
          break;
        }
        sm100::tc_fence_after();
        const uint32_t d_tmem = tmem_base + as * TN;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
          if (!__all_sync(0xffffffffu, sm100::mbar_wait(&full[s], ph))) {
            if (leader) sm100::report_timeout(a.status, 12);
            ok = false;
            break;
          }
          sm100::tc_fence_after();
          const uint32_t a_addr = sm100::smem_u32(smem + s * STAGE_BYTES);
          const uint32_t b_addr = a_addr + A_BYTES;
          if (leader) {
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              const uint64_t adesc = a.x_km ? sm100::umma_desc_mn_sw128(a_addr + k * (UMMA_K * 128), BK * 128)
                                            : sm100::umma_desc_k_sw128(a_addr + k * (UMMA_K * 2));
              // [N, K] weights are K-major like x; [K, N] weights are MN-major: 16 k-rows of 128
              // bytes per step, 64-column atoms BK*128 bytes apart
              const uint64_t bdesc = a.w_kn ? sm100::umma_desc_mn_sw128(b_addr + k * (UMMA_K * 128), BK * 128)
                                            : sm100::umma_desc_k_sw128(b_addr + k * (UMMA_K * 2));
              sm100::umma_f16_ss(d_tmem, adesc, bdesc, idesc, (kb > 0 || k > 0) ? 1u : 0u);
            }
            sm100::umma_commit(&empty[s]);  // stage reusable once these MMAs have read it
          }
          __syncwarp();
        }
        if (ok && leader) sm100::umma_commit(&acc_full[as]);
        __syncwarp();
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..9)
    const int q = warp & 3;  // TMEM lane quadrant this warp may read
    uint32_t tile_iter = 0;
    const bool vec_ok = (a.N % 8) == 0 && (reinterpret_cast<uintptr_t>(a.out) & 15u) == 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++tile_iter) {
      const int m0 = (tile % a.tiles_m) * BM, n0 = (tile / a.tiles_m) * TN;
      const uint32_t as = tile_iter % ACC_STAGES, aph = (tile_iter / ACC_STAGES) & 1;
      if (!sm100::mbar_wait(&acc_full[as], aph)) { sm100::report_timeout(a.status, 13); break; }
      sm100::tc_fence_after();
      const int row = m0 + q * 32 + lane;
      const uint32_t t_base = tmem_base + as * TN + (static_cast<uint32_t>(q * 32) << 16);
      epilogue_tile<BF16, G::CHUNKS>(a, t_base, row, n0, vec_ok, ((warp - 2) >> 2) * G::CHUNKS);
      sm100::tc_fence_before();
      __syncwarp();
      if (lane == 0) sm100::mbar_arrive(&acc_empty[as]);
    }
  }

  sm100::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    sm100::tc_fence_after();
    sm100::tmem_dealloc(tmem_base, G::TMEM);
  }
}

// ---------------------------------------------------------------- CTA-pair variant
// Two CTAs of a cluster (one TPC) share a 256 x 256 output tile: each owns 128 of its rows
// (its own accumulator in its own TMEM) and stages 128 rows of x plus HALF of the weight tile;
// tcgen05.mma.cta_group::2 reads both halves, so every SM fetches 32 KB per k-block instead of
// 48 KB for the same math -- operand bandwidth from L2, not the tensor pipe, limited the 1-CTA
// form.  The even CTA of the pair issues the MMAs; completion is multicast to both CTAs'
// barriers; each CTA loads its own tiles (no multicast load).
constexpr int P_BM = 256, P_BN = 256;                 // pair tile
constexpr int P_A_BYTES = 128 * BK * 2;               // per CTA: 128 rows of x
constexpr int P_B_BYTES = 128 * BK * 2;               // per CTA: 128 of the 256 weight rows
constexpr int P_STAGE_BYTES = P_A_BYTES + P_B_BYTES;  // 32 KB
constexpr int P_STAGES = 6;
constexpr size_t P_SMEM_BYTES = static_cast<size_t>(P_STAGES) * P_STAGE_BYTES + 1024 + 256;

template <bool BF16>
__global__ void __launch_bounds__(NUM_THREADS, 1) gemm_epilogue_pair_kernel(const __grid_constant__ GemmArgs a) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + P_STAGES * P_STAGE_BYTES);
  uint64_t* empty = full + P_STAGES;
  uint64_t* acc_full = empty + P_STAGES;
  uint64_t* acc_empty = acc_full + ACC_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + ACC_STAGES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = sm100::cluster_ctarank();     // 0 = leader (issues MMAs), 1 = peer
  const int pair = static_cast<int>(blockIdx.x >> 1), n_pairs = static_cast<int>(gridDim.x >> 1);

  if (warp == 0 && lane == 0) {
    sm100::prefetch_tensormap(&a.tmap_a);
    sm100::prefetch_tensormap(&a.tmap_b);
    for (int s = 0; s < P_STAGES; ++s) {
      sm100::mbar_init(&full[s], 1);    // used in the leader only: its producer's arrive.expect_tx
      sm100::mbar_init(&empty[s], 1);   // one multicast commit per phase, in both CTAs
    }
    for (int s = 0; s < ACC_STAGES; ++s) {
      sm100::mbar_init(&acc_full[s], 1);   // multicast commit, both CTAs
      sm100::mbar_init(&acc_empty[s], 2 * EPI_WARPS);  // leader only: the epilogue warps of both CTAs
    }
    sm100::fence_barrier_init();
  }
  if (warp == 1) {
    sm100::tmem_alloc_pair(tmem_slot, TMEM_COLS);
    sm100::tmem_relinquish_pair();
  }
  sm100::tc_fence_before();
  sm100::cluster_sync_all();   // both CTAs' barriers exist before anything signals them remotely
  sm100::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Programmatic dependent launch (see the 1-CTA kernel): set-up above overlaps the previous
  // kernel's tail, global memory is touched only after it has completed.
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");

  const int num_tiles = a.tiles_m * a.tiles_n;       // 256 x 256 tiles
  const int kblocks = (a.K + BK - 1) / BK;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += n_pairs) {
        const int m0 = (tile % a.tiles_m) * P_BM + static_cast<int>(rank) * 128;
        const int n0 = (tile / a.tiles_m) * P_BN + static_cast<int>(rank) * 128;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const uint32_t s = it % P_STAGES, ph = (it / P_STAGES) & 1;
          if (!sm100::mbar_wait(&empty[s], ph ^ 1)) { sm100::report_timeout(a.status, 30); ok = false; break; }
          if (rank == 0) sm100::mbar_arrive_expect_tx(&full[s], 2 * P_STAGE_BYTES);  // both CTAs' bytes
          unsigned char* st = smem + s * P_STAGE_BYTES;
          if (!a.x_km) {
            sm100::tma_load_2d_pair(st, &a.tmap_a, kb * BK, m0, &full[s]);
          } else {   // [K, M]: this CTA's 128 rows of the tile as two boxes of 64 k-rows
            sm100::tma_load_2d_pair(st, &a.tmap_a, m0, kb * BK, &full[s]);
            sm100::tma_load_2d_pair(st + BK * 128, &a.tmap_a, m0 + 64, kb * BK, &full[s]);
          }
          if (!a.w_kn) {
            sm100::tma_load_2d_pair(st + P_A_BYTES, &a.tmap_b, kb * BK, n0, &full[s]);
          } else {   // [K, N]: this CTA's 128 columns of N as two boxes of 64 k-rows
            sm100::tma_load_2d_pair(st + P_A_BYTES, &a.tmap_b, n0, kb * BK, &full[s]);
            sm100::tma_load_2d_pair(st + P_A_BYTES + BK * 128, &a.tmap_b, n0 + 64, kb * BK, &full[s]);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    // The whole warp runs the loop convergently and one elected lane issues the tcgen05
    // instructions, so the operand descriptors stay in uniform registers.
    if (rank == 0) {
      const bool leader = sm100::elect_one();
      const uint32_t idesc = sm100::umma_idesc_f16(P_BM, P_BN, BF16, a.x_km != 0, a.w_kn != 0);
      uint32_t it = 0, tile_iter = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += n_pairs, ++tile_iter) {
        const uint32_t as = tile_iter % ACC_STAGES, aph = (tile_iter / ACC_STAGES) & 1;
        if (!__all_sync(0xffffffffu, sm100::mbar_wait(&acc_empty[as], aph ^ 1))) {
          if (leader) sm100::report_timeout(a.status, 31);
          break;
        }
        sm100::tc_fence_after();
        const uint32_t d_tmem = tmem_base + as * BN;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const uint32_t s = it % P_STAGES, ph = (it / P_STAGES) & 1;
          if (!__all_sync(0xffffffffu, sm100::mbar_wait(&full[s], ph))) {
            if (leader) sm100::report_timeout(a.status, 32);
            ok = false;
            break;
          }
          sm100::tc_fence_after();
          const uint32_t a_addr = sm100::smem_u32(smem + s * P_STAGE_BYTES);
          const uint32_t b_addr = a_addr + P_A_BYTES;
          if (leader) {
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              const uint64_t adesc = a.x_km ? sm100::umma_desc_mn_sw128(a_addr + k * (UMMA_K * 128), BK * 128)
                                            : sm100::umma_desc_k_sw128(a_addr + k * (UMMA_K * 2));
              const uint64_t bdesc = a.w_kn ? sm100::umma_desc_mn_sw128(b_addr + k * (UMMA_K * 128), BK * 128)
                                            : sm100::umma_desc_k_sw128(b_addr + k * (UMMA_K * 2));
              sm100::umma_f16_ss_pair(d_tmem, adesc, bdesc, idesc, (kb > 0 || k > 0) ? 1u : 0u);
            }
            sm100::umma_commit_pair(&empty[s], 3);   // frees the stage in both CTAs
          }
          __syncwarp();
        }
        if (ok && leader) sm100::umma_commit_pair(&acc_full[as], 3);
        __syncwarp();
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..9, both CTAs)
    const int q = warp & 3;
    uint32_t tile_iter = 0;
    const bool vec_ok = (a.N % 8) == 0 && (reinterpret_cast<uintptr_t>(a.out) & 15u) == 0;
    const uint32_t leader_acc_empty = sm100::mapa_u32(sm100::smem_u32(&acc_empty[0]), 0);
    for (int tile = pair; tile < num_tiles; tile += n_pairs, ++tile_iter) {
      const int m0 = (tile % a.tiles_m) * P_BM + static_cast<int>(rank) * 128, n0 = (tile / a.tiles_m) * P_BN;
      const uint32_t as = tile_iter % ACC_STAGES, aph = (tile_iter / ACC_STAGES) & 1;
      if (!sm100::mbar_wait(&acc_full[as], aph)) { sm100::report_timeout(a.status, 33); break; }
      sm100::tc_fence_after();
      const int row = m0 + q * 32 + lane;
      const uint32_t t_base = tmem_base + as * BN + (static_cast<uint32_t>(q * 32) << 16);
      epilogue_tile<BF16>(a, t_base, row, n0, vec_ok, ((warp - 2) >> 2) * EPI_CHUNKS);
      sm100::tc_fence_before();
      __syncwarp();
      if (lane == 0) sm100::mbar_arrive_remote(leader_acc_empty + as * 8);   // the leader's barrier, from either CTA
    }
  }

  sm100::tc_fence_before();
  sm100::cluster_sync_all();   // neither CTA leaves while its peer may still signal it
  if (warp == 1) {
    sm100::tc_fence_after();
    sm100::tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

}  // namespace

// Row-major 2-D tensor [rows, cols] of 16-bit elements, box = box_cols x box_rows, 128-byte swizzle.
int make_tensor_map_2d(CUtensorMap* map, const void* base, int is_bf16, int64_t rows, int64_t cols, int box_rows,
                       int box_cols) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) { set_error("cuTensorMapEncodeTiled is not available from the driver"); return CDR_ERR_CUDA; }
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * 2};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                  const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed with %d", static_cast<int>(r)); return CDR_ERR_CUDA; }
  return CDR_OK;
}

// Row-major 3-D tensor [d2, d1, d0] (d0 contiguous) of 16-bit elements, box = box0 x box1 x 1,
// 128-byte swizzle; rows beyond d1 read as zeros.
int make_tensor_map_3d(CUtensorMap* map, const void* base, int is_bf16, int64_t d0, int64_t d1, int64_t d2,
                       int box0, int box1) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) { set_error("cuTensorMapEncodeTiled is not available from the driver"); return CDR_ERR_CUDA; }
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(d0), static_cast<cuuint64_t>(d1), static_cast<cuuint64_t>(d2)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(d0) * 2, static_cast<cuuint64_t>(d0) * d1 * 2};
  const cuuint32_t box[3] = {static_cast<cuuint32_t>(box0), static_cast<cuuint32_t>(box1), 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                  const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled (3-D) failed with %d", static_cast<int>(r)); return CDR_ERR_CUDA; }
  return CDR_OK;
}

// Same tensor without swizzle: the layout a TMA store reads from a plain row-major shared-memory box.
int make_tensor_map_3d_plain(CUtensorMap* map, const void* base, int is_bf16, int64_t d0, int64_t d1, int64_t d2,
                             int box0, int box1) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) { set_error("cuTensorMapEncodeTiled is not available from the driver"); return CDR_ERR_CUDA; }
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(d0), static_cast<cuuint64_t>(d1), static_cast<cuuint64_t>(d2)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(d0) * 2, static_cast<cuuint64_t>(d0) * d1 * 2};
  const cuuint32_t box[3] = {static_cast<cuuint32_t>(box0), static_cast<cuuint32_t>(box1), 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                  const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled (3-D, plain) failed with %d", static_cast<int>(r)); return CDR_ERR_CUDA; }
  return CDR_OK;
}

int launch_gemm_epilogue(const cdr_tensor* ins, int n_in, const cdr_tensor* outs, int n_out,
                         const cdr_gemm_params* p, cudaStream_t stream) {
  if (!p) { set_error("gemm_epilogue: params is null"); return CDR_ERR_BAD_ARG; }
  const int want_in = 2 + (p->has_bias ? 1 : 0) + (p->gate_input ? 1 : 0);
  if (n_in != want_in || n_out != 1) {
    set_error("gemm_epilogue: expects %d inputs and 1 output, got %d and %d", want_in, n_in, n_out);
    return CDR_ERR_BAD_ARG;
  }
  if (p->activation != CDR_ACT_NONE && p->activation != CDR_ACT_RELU) {
    set_error("gemm_epilogue: unknown activation %d", p->activation);
    return CDR_ERR_UNSUPPORTED;
  }
  const cdr_tensor &x = ins[0], &w = ins[1], &out = outs[0];
  if (x.rank < 1 || w.rank != 2) { set_error("gemm_epilogue: x needs rank >= 1 and W rank 2"); return CDR_ERR_BAD_ARG; }
  const bool x_km = p->x_layout == CDR_X_KM;
  if (p->x_layout != CDR_X_MK && !x_km) { set_error("gemm_epilogue: unknown x layout %d", p->x_layout); return CDR_ERR_BAD_ARG; }
  if (x_km && x.rank != 2) { set_error("gemm_epilogue: [K, M] x must have rank 2"); return CDR_ERR_BAD_ARG; }
  const int64_t K = x_km ? x.shape[0] : x.shape[x.rank - 1];
  const int64_t M = x_km ? x.shape[1] : (K ? numel(x) / K : 0);
  const bool w_kn = p->weight_layout == CDR_W_KN;
  if (p->weight_layout != CDR_W_NK && !w_kn) { set_error("gemm_epilogue: unknown weight layout %d", p->weight_layout); return CDR_ERR_BAD_ARG; }
  const int64_t N = w.shape[w_kn ? 1 : 0];
  if (w.shape[w_kn ? 0 : 1] != K) {
    set_error("gemm_epilogue: x has K=%lld, W has K=%lld", (long long)K, (long long)w.shape[w_kn ? 0 : 1]);
    return CDR_ERR_BAD_ARG;
  }
  if (numel(out) != M * N) { set_error("gemm_epilogue: output must hold %lld elements", (long long)(M * N)); return CDR_ERR_BAD_ARG; }
  const int dt = x.dtype;
  if (dt != CDR_BF16 && dt != CDR_F16) { set_error("gemm_epilogue: dtype %d unsupported (bf16 and f16 only)", dt); return CDR_ERR_UNSUPPORTED; }
  if (w.dtype != dt || out.dtype != dt || (p->has_bias && ins[2].dtype != dt)) {
    set_error("gemm_epilogue: x, W, bias and output must share one dtype");
    return CDR_ERR_UNSUPPORTED;
  }
  if (!is_contiguous(x) || !is_contiguous(w) || !is_contiguous(out) || (p->has_bias && !is_contiguous(ins[2]))) {
    set_error("gemm_epilogue: tensors must be contiguous");
    return CDR_ERR_BAD_ARG;
  }
  if (p->has_bias && numel(ins[2]) != N) { set_error("gemm_epilogue: bias must hold N=%lld elements", (long long)N); return CDR_ERR_BAD_ARG; }
  if (M == 0 || N == 0) return CDR_OK;
  if (K == 0) { set_error("gemm_epilogue: K == 0"); return CDR_ERR_UNSUPPORTED; }
  if (!x.data || !w.data || !out.data || (p->has_bias && !ins[2].data)) { set_error("gemm_epilogue: null pointer"); return CDR_ERR_BAD_ARG; }
  if (K % 8 != 0 && !(x_km && w_kn)) { set_error("gemm_epilogue: K=%lld must be a multiple of 8 (16-byte row pitch for TMA)", (long long)K); return CDR_ERR_UNSUPPORTED; }
  if (x_km && M % 8 != 0) { set_error("gemm_epilogue: M=%lld must be a multiple of 8 for [K, M] x", (long long)M); return CDR_ERR_UNSUPPORTED; }
  if (w_kn && N % 8 != 0) { set_error("gemm_epilogue: N=%lld must be a multiple of 8 for [K, N] weights", (long long)N); return CDR_ERR_UNSUPPORTED; }
  if (!aligned16(x.data) || !aligned16(w.data)) { set_error("gemm_epilogue: x and W must be 16-byte aligned"); return CDR_ERR_MISALIGNED; }
  if (M > 0x7fffffff || N > 0x7fffffff || K > 0x7fffffff) { set_error("gemm_epilogue: extent too large"); return CDR_ERR_UNSUPPORTED; }

  GemmArgs a;
  if (int rc = x_km ? make_tensor_map_2d(&a.tmap_a, x.data, dt == CDR_BF16, K, M, BK, 64)
                    : make_tensor_map_2d(&a.tmap_a, x.data, dt == CDR_BF16, M, K, BM, BK)) return rc;
  a.x_km = x_km ? 1 : 0;
  // [K, N] weights: rows are k, 64 columns of N (128 bytes) per box, BK rows
  if (int rc = w_kn ? make_tensor_map_2d(&a.tmap_b, w.data, dt == CDR_BF16, K, N, BK, 64)
                    : make_tensor_map_2d(&a.tmap_b, w.data, dt == CDR_BF16, N, K, BN, BK)) return rc;
  a.w_kn = w_kn ? 1 : 0;
  a.bias = p->has_bias ? ins[2].data : nullptr;
  a.gate = nullptr;
  if (p->gate_input) {
    const cdr_tensor& gt = ins[want_in - 1];
    if (gt.dtype != dt || numel(gt) != M * N || !is_contiguous(gt) || !gt.data) {
      set_error("gemm_epilogue: the gate tensor must be contiguous, of the output's dtype and element count");
      return CDR_ERR_BAD_ARG;
    }
    a.gate = gt.data;
  }
  a.out = out.data;
  a.M = static_cast<int>(M); a.N = static_cast<int>(N); a.K = static_cast<int>(K);
  a.relu = p->activation == CDR_ACT_RELU;
  a.is_bf16 = dt == CDR_BF16;
  a.status = device_status_ptr();
  int dev = 0;
  CDR_CUDA_TRY(cudaGetDevice(&dev));
  static bool configured_dev[64] = {false};
  bool& configured = configured_dev[dev & 63];
  if (!configured) {
    CDR_CUDA_TRY(cudaFuncSetAttribute(gemm_epilogue_kernel<true, 256>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(Tile1<256>::SMEM)));
    CDR_CUDA_TRY(cudaFuncSetAttribute(gemm_epilogue_kernel<false, 256>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(Tile1<256>::SMEM)));
    CDR_CUDA_TRY(cudaFuncSetAttribute(gemm_epilogue_kernel<true, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(Tile1<128>::SMEM)));
    CDR_CUDA_TRY(cudaFuncSetAttribute(gemm_epilogue_kernel<false, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(Tile1<128>::SMEM)));
    CDR_CUDA_TRY(cudaFuncSetAttribute(gemm_epilogue_pair_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(P_SMEM_BYTES)));
    CDR_CUDA_TRY(cudaFuncSetAttribute(gemm_epilogue_pair_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(P_SMEM_BYTES)));
    configured = true;
  }

  static const bool pdl = getenv("CDR_DISABLE_PDL") == nullptr;
  // Few large tiles leave most SMs idle: when the 256 x 256 pair tiles fill less than half of the
  // CTA pairs and 128 x 128 tiles would still fit in one wave, run the 1-CTA kernel on 128 x 128
  // tiles instead (a 1024 x 1024 x 4096 product: 16 pair tiles on 74 pairs, or 64 tiles on 148 SMs).
  const int64_t pair_tiles = ((M + P_BM - 1) / P_BM) * ((N + P_BN - 1) / P_BN);
  const int64_t small_tiles = ((M + BM - 1) / BM) * ((N + 127) / 128);
  const bool narrow = N >= 128 && 2 * pair_tiles < sm_count() / 2 && small_tiles <= sm_count() && small_tiles > 2 * pair_tiles;
  if (M >= P_BM && N >= P_BN && !narrow) {
    // CTA-pair kernel: 256 x 256 tiles, clusters of two CTAs, at most one cluster per TPC.
    // Each CTA stages only 128 of the tile's 256 weight rows: the W box is 64 x 128 here.
    if (!w_kn)
      if (int rc = make_tensor_map_2d(&a.tmap_b, w.data, dt == CDR_BF16, N, K, 128, BK)) return rc;
    a.tiles_m = static_cast<int>((M + P_BM - 1) / P_BM);
    a.tiles_n = static_cast<int>((N + P_BN - 1) / P_BN);
    const int64_t tiles = static_cast<int64_t>(a.tiles_m) * a.tiles_n;
    int pairs = sm_count() / 2;
    if (pairs > tiles) pairs = static_cast<int>(tiles);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(2 * pairs), 1, 1);
    cfg.blockDim = dim3(NUM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = P_SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    if (dt == CDR_BF16) CDR_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemm_epilogue_pair_kernel<true>, a));
    else CDR_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemm_epilogue_pair_kernel<false>, a));
    return CDR_OK;
  }

  const int tn = narrow ? 128 : BN;
  if (narrow && !w_kn)     // the weight box follows the tile: 128 rows of W per k-block
    if (int rc = make_tensor_map_2d(&a.tmap_b, w.data, dt == CDR_BF16, N, K, 128, BK)) return rc;
  a.tiles_m = static_cast<int>((M + BM - 1) / BM);
  a.tiles_n = static_cast<int>((N + tn - 1) / tn);
  const int64_t tiles = static_cast<int64_t>(a.tiles_m) * a.tiles_n;
  int grid = sm_count();
  if (grid > tiles) grid = static_cast<int>(tiles);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
  cfg.blockDim = dim3(NUM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = narrow ? Tile1<128>::SMEM : Tile1<256>::SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (narrow) {
    if (dt == CDR_BF16) CDR_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemm_epilogue_kernel<true, 128>, a));
    else CDR_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemm_epilogue_kernel<false, 128>, a));
    return CDR_OK;
  }
  if (dt == CDR_BF16) CDR_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemm_epilogue_kernel<true, 256>, a));
  else CDR_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemm_epilogue_kernel<false, 256>, a));
  return CDR_OK;
}

}  // namespace cdr
