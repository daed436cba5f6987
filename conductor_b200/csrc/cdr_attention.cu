// K5 -- fused scaled-dot-product attention:  O = softmax(Q K^T * scale [+ causal mask]) V.
//
// Reference definitions: the three-phase kernels of choreo-op/attention-gcu-only-test.co:15-134 and
// efficientattention-gcu-only-test.co:13-126, and the per-row online-softmax recurrence of
// choreo-op/flashattention-gcu-only-test.co:75-122 (d_i = d_prev*e^(m_prev-m) + e^(s-m)); the
// executed path is eager torch.nn.functional.scaled_dot_product_attention in bf16.
//
// Tensor-core bound.  Persistent CTAs, one per SM, each walking a fixed, balanced sequence of
// (batch*head, 256-query) tiles, so that the loads and first scores of a tile overlap the output
// phase of the previous one.  A tile is handled as two 128-row halves A and B that share every
// K/V block (halving operand traffic per flop) and ping-pong on the tensor core: while the softmax
// warps of one half work, the MMAs of the other half run.
//   warp 0      TMA producer: both Q halves per tile, K_j and V_j through one 4-stage ring that
//               never resets across tiles
//   warp 1      MMA issuer:  S_h = Q_h K_j^T (fp32 in TMEM) and O_h += P_h V_j, where P_h is
//               read straight from TMEM (it overwrites the S_h columns as packed bf16).  The whole
//               warp runs the loop convergently and an elected lane issues, which keeps the
//               operand descriptors in uniform registers (a single-lane branch cost ~95 cycles
//               per MMA, more than the 64 cycles a 128x128x16 MMA executes in)
//   warps 2-3   idle: they complete the control warp group so that setmaxnreg can hand its
//               registers (80 per thread kept) to the softmax groups (208 per thread, no spills)
//   warps 4-7   softmax of half A, warps 8-11 of half B (and the tile's epilogue: O / l packed into a
//               2 KB shared-memory stage per warp and written by tiled TMA stores): one query row per thread; tcgen05.ld
//               the S row, running max (3-input max) / sum in the log2 domain, P = exp2(..) with
//               two-lane fp32 instructions (a cubic on the FMA pipes can take pairs off the
//               special-function unit, CDR_ATT_EMU, but no share of it paid off), stored back to TMEM with tcgen05.st; the O
//               accumulator stays in TMEM and is rescaled only when the
//               running max grew by more than 2^8 (exact after the final division)
// TMEM columns: S_A 0-127, S_B 128-255, O_A 256-383, O_B 384-511.  MMAs of one CTA execute in
// issue order, so reusing the S_h columns for S_h(j+1) after P_h(j) needs no extra barrier.
// Tiles are handed out dynamically: the producer warp takes the next tile index from a counter in
// global scratch (one atomic per tile, fetched one tile ahead) and publishes it to the other warps
// through a small shared-memory ring.  The index order keeps the heads that are in flight at any
// time few -- groups of about (SMs / query tiles per head) heads, so that the K/V of a head is read
// from HBM once and then served by L2 to the CTAs working on its other query tiles -- and inside
// a group runs the triangular causal work heaviest first, which leaves only light tiles for the
// tail.  No load is multicast; every wait is bounded and reports through the device status word.
// The softmax warps compute P = exp2(s*c - m_ref) for block j > 0 against the reference maximum
// they already hold, accumulating the block's own maximum on the side; only when that maximum
// exceeds the reference by more than 2^8 (rare after the first blocks) is the accumulator rescaled
// and P recomputed.  This takes the row-max pass off the softmax -> MMA critical chain.
// Measured alternatives that lost: a polling issuer that lets a half run into the next tile (-8 %), 64-key blocks
// with P double-buffered beside S (-50 %: the tensor core accepts about one MMA per 90 cycles
// whatever its N, so halving N halves the rate), 16 softmax warps, two threads per row (-17 %), P handed
// over in two parts of 64 keys so that half of P.V starts early (-1.5 %); sixteen softmax warps with
// the key columns of a row split over two threads that agree on the reference maximum only in a
// tile's first block and on a rescale (equal at S=8192, -14 % at S=2048: four warps per scheduler
// contend for the special-function unit whenever the two halves' exp passes overlap); bf16 packing
// by integer add + byte permute instead of cvt (no change: the conversion runs on the half-rate
// ALU pipe, not on the special-function unit); polynomial exp2 for 2/8 or 4/8 of the pairs with
// sixteen warps (-1 %, -6 %: with half-rate f32x2 arithmetic the cubic costs more issue cycles than
// the special-function time it frees); Q buffers and barriers per half with the first scores of
// the next tile issued for half A as soon as it finishes its last block of the current one, so that
// under a causal mask its softmax runs beside half B's last block (-3 % on every shape, the
// non-causal ones included: the longer issue loop of the MMA warp costs more than the overlap gains);
// an epilogue that keeps the next chunk's tcgen05.ld in flight while the current one is stored (-2 %).
// Structural variants, all measured on one box against this kernel (193 / 1052 / 617 us at C5, S=8192
// non-causal, S=8192 causal) and dropped: (1) the two halves as independent chains with their own
// 128-row work items, Q buffer, two-slot K/V ring, TMA warp and MMA warp: 206 / 1219 / 696 (a K/V block
// is then fetched from L2 once per chain; with those fetches halved for diagnosis still 201 / 1110 / 657);
// (2) P handed over through shared memory in the K-major swizzled operand layout instead of over S in
// tensor memory, so that S(j+1) is issued as soon as S(j) is in registers and runs under the
// exponentials of block j, one MMA warp per half, a three-slot ring in consumption order: the wait for
// the scores falls from ~1700 to ~230 cycles per block, but the total is 195.6 / 1021 / 607 -- every
// MMA then reads both operands from shared memory, P adds 64 KB of writes per block pair, and the
// halves' exponential passes fall into step; making the paired warps of a scheduler take turns at the
// exponentials made it 301 / 1723 / 1044; (3) this kernel with one MMA-issuing warp per half:
// 207 / 1265 / 692.  With the exponentials replaced by a multiplication (wrong results, diagnosis
// only) this kernel runs 183 / 1061 / 614: the exponential pass itself shrinks (1595 -> 895 cycles per
// block), but the wait for the scores grows by as much -- the MMA warp, which serves the two halves in
// turn and needs ~2000 cycles per group of 16 MMAs all told, sets the pace, not the special-function unit.
// Micro-benchmarks beside it: a 128x128x16 MMA executes in 64.6 cycles whatever the source and layout of
// its operands (52.7 at N=64, 128.6 at N=256); the issuing thread stays blocked while the pipe works
// (a batch of 16 MMAs returns after 935 cycles: about one and a half MMAs are queued), and the commit
// is seen about 210 cycles after the last MMA was issued.  Per block and half the chain is therefore
// softmax (~2100 cycles) + P.V and the next scores (1034) + hand-over latency; taking the MMAs off it
// needs S and P side by side in tensor memory, which two halves at head dimension 128 leave no room for.
// What did pay in the epilogue: 256-bit stores (two per 32 columns instead of four 128-bit ones), +4 %,
// and then handing the stores to the TMA unit from per-warp shared-memory stages, +1.5 % more.
#include <cuda.h>
#include <math.h>

#include "cdr_common.cuh"
#include "cdr_sm100.cuh"

// Cycle accounting for development (-DCDR_ATT_PROF): one thread per role adds the clock64 time
// it spends in each wait or phase to a per-CTA table in shared memory, written to the tail of the
// scratch buffer at exit.  Compiled out by default.
#ifdef CDR_ATT_PROF
#define PROF_SLOTS 128
#define PROF_BEGIN(cond) long long prof_t0_ = (cond) ? clock64() : 0
#define PROF_MARK(cond) if (cond) prof_t0_ = clock64()
#define PROF_ADD(cond, idx) do { if (cond) { const long long now_ = clock64(); prof_tab[(idx)] += now_ - prof_t0_; prof_t0_ = now_; } } while (0)
#define PROF_COUNT(cond, idx) do { if (cond) prof_tab[(idx)] += 1; } while (0)
#else
#define PROF_SLOTS 0
#define PROF_BEGIN(cond)
#define PROF_MARK(cond)
#define PROF_ADD(cond, idx)
#define PROF_COUNT(cond, idx)
#endif

namespace cdr {

int make_tensor_map_3d(CUtensorMap* map, const void* base, int is_bf16, int64_t d0, int64_t d1, int64_t d2,
                       int box0, int box1);
int make_tensor_map_3d_plain(CUtensorMap* map, const void* base, int is_bf16, int64_t d0, int64_t d1, int64_t d2,
                             int box0, int box1);

namespace {

constexpr int BQ = 256, BH_ROWS = 128, BKV = 128;   // query tile, rows per half, keys per block
// Roles aligned to warp groups so that setmaxnreg can move registers from the control warps to the
// softmax warps: group 0 = TMA warp, MMA warp and two idle warps; groups 1, 2 = softmax of half A, B.
constexpr int ATT_THREADS = 384;
constexpr int SOFTMAX_WARP0 = 4;
constexpr int REGS_CONTROL = 80, REGS_SOFTMAX = 208;   // 128*80 + 256*208 <= 384*168, the CTA's allocation at launch
constexpr int TMEM_S = 0, TMEM_O = 256, ATT_TMEM_COLS = 512;   // + 128 * half
constexpr float kRescaleThreshold = 8.0f;  // log2 units

struct AttnArgs {
  CUtensorMap tmap_q, tmap_k, tmap_v;  // [BH, S, D] each, box 64 x 128 x 1
  CUtensorMap tmap_o;                  // the output, [BH, S, D], box 32 x 32 x 1, no swizzle (epilogue stores)
  void* out;                            // [BH, S, D]
  unsigned int* next_tile;              // global scratch: tiles handed out beyond the first one per CTA
  int S, BH, n_qtiles;
  int group_heads, total_tiles;         // heads per scheduling group; BH * n_qtiles
  float scale_log2;                     // scale * log2(e)
  int causal;
  int* status;
};

constexpr int KV_STAGES = 4;   // one ring for K and V tiles: K_0 V_0 K_1 V_1 ... (4 measured as fast as 5)
constexpr int TILE_SLOTS = 4;  // ring of tile indices from the producer warp to the MMA and softmax warps
constexpr int TILE_READERS = 9;  // the MMA warp and the eight softmax warps release a slot

template <int HD>
struct AttnSmem {
  static constexpr int TILE_BYTES = 128 * HD * 2;      // one Q half, K block or V block
  static constexpr int Q_OFF = 0;                      // 2 halves
  static constexpr int KV_OFF = 2 * TILE_BYTES;        // KV_STAGES tiles
  static constexpr int BAR_OFF = KV_OFF + KV_STAGES * TILE_BYTES;
  static constexpr int STAGE_OFF = BAR_OFF + 256;            // 8 softmax warps x (32 rows x 64 bytes): epilogue store stages
  static constexpr int STAGE_BYTES = 8 * 32 * 64;
  static constexpr int PROF_OFF = STAGE_OFF + STAGE_BYTES;
  static constexpr size_t TOTAL = PROF_OFF + PROF_SLOTS * 8 + 1024;
};

// barrier indices; ring barriers are indexed by stage, the others by half
enum { B_QFULL = 0, B_QEMPTY = 1, B_FULL = 2, B_EMPTY = B_FULL + KV_STAGES, B_SFULL = B_EMPTY + KV_STAGES, B_PFULL = B_SFULL + 2,
       B_PVDONE = B_PFULL + 2, B_OFREE = B_PVDONE + 2, B_TFULL = B_OFREE + 2, B_TEMPTY = B_TFULL + TILE_SLOTS,
       B_COUNT = B_TEMPTY + TILE_SLOTS };

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

#ifndef CDR_ATT_EMU
#define CDR_ATT_EMU 0   // pairs of every 8 whose exp2 runs on the FMA pipes (0: measured best on this kernel)
#endif

// ---- two fp32 lanes per instruction (fma/add/sub .f32x2) and the three-input max of sm_100
__device__ __forceinline__ uint64_t pack2(float a, float b) { uint64_t r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b)); return r; }
__device__ __forceinline__ void unpack2(uint64_t v, float& a, float& b) { asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v)); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) { uint64_t d; asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c)); return d; }
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) { uint64_t d; asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d; }
__device__ __forceinline__ uint64_t sub2(uint64_t a, uint64_t b) { uint64_t d; asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d; }
__device__ __forceinline__ float max3(float a, float b, float c) { float d; asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c)); return d; }

// 2^x for a pair on the FMA pipes instead of the special-function unit: x = n + f with n the
// nearest integer (magic-number rounding) and f in [-0.5, 0.5]; 2^f by a cubic (max relative error
// 7.5e-5, far inside the 2^-9 of the 16-bit P it feeds); n goes straight into the exponent field.
// Inputs are clamped to -125 so the exponent cannot wrap.
__device__ __forceinline__ void poly_exp2_pair(uint64_t x, float& p0, float& p1) {
  float x0, x1;
  unpack2(x, x0, x1);
  x = pack2(fmaxf(x0, -125.0f), fmaxf(x1, -125.0f));
  const uint64_t magic = pack2(12582912.0f, 12582912.0f);
  const uint64_t t = add2(x, magic);
  const uint64_t f = sub2(x, sub2(t, magic));
  uint64_t r = fma2(pack2(0.055171459913253784f, 0.055171459913253784f), f, pack2(0.2426108568906784f, 0.2426108568906784f));
  r = fma2(r, f, pack2(0.6932609677314758f, 0.6932609677314758f));
  r = fma2(r, f, pack2(0.9999281167984009f, 0.9999281167984009f));
  float t0, t1, r0, r1;
  unpack2(t, t0, t1);
  unpack2(r, r0, r1);
  p0 = __uint_as_float(__float_as_uint(r0) + (__float_as_uint(t0) << 23));
  p1 = __uint_as_float(__float_as_uint(r1) + (__float_as_uint(t1) << 23));
}

template <bool BF16>
__device__ __forceinline__ uint32_t pack_pair(float a, float b) {
  if (BF16) { __nv_bfloat162 t = __floats2bfloat162_rn(a, b); return *reinterpret_cast<uint32_t*>(&t); }
  __half2 t = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&t);
}

// P = exp2(s*c - m) for one row's 128 scores, packed to 16-bit pairs and stored over the S columns the
// row just read (`p_taddr`); row sums accumulate in two fp32 lanes.  EMU of every 8 pairs take the polynomial path,
// the rest the special-function unit.
// With WITH_MAX the maximum of the raw scores is accumulated alongside (four independent chains) and returned.
template <bool BF16, int EMU, bool WITH_MAX>
__device__ __forceinline__ float store_p(uint32_t (&sr)[4][32], float scale_log2, float neg_m, float& l0, float& l1, uint32_t p_taddr) {
  const uint64_t scale2 = pack2(scale_log2, scale_log2), negm2 = pack2(neg_m, neg_m);
  uint64_t lsum4[4] = {pack2(l0, l1), pack2(0.0f, 0.0f), pack2(0.0f, 0.0f), pack2(0.0f, 0.0f)};   // independent chains
  float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint32_t pw[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float p0, p1;
      const uint64_t x = fma2(pack2(__uint_as_float(sr[c][2 * i]), __uint_as_float(sr[c][2 * i + 1])), scale2, negm2);
      if (WITH_MAX) mx[i & 1] = max3(mx[i & 1], __uint_as_float(sr[c][2 * i]), __uint_as_float(sr[c][2 * i + 1]));
      if ((i & 7) < EMU) {
        poly_exp2_pair(x, p0, p1);
      } else {
        float x0, x1;
        unpack2(x, x0, x1);
        p0 = fast_exp2(x0);
        p1 = fast_exp2(x1);
      }
      lsum4[i & 3] = add2(lsum4[i & 3], pack2(p0, p1));
      pw[i] = pack_pair<BF16>(p0, p1);
    }
    sm100::tmem_st16(p_taddr + c * 16, pw);
  }
  unpack2(add2(add2(lsum4[0], lsum4[1]), add2(lsum4[2], lsum4[3])), l0, l1);
  return fmaxf(mx[0], mx[1]);
}

// One (batch*head, 256-query) tile of this CTA's sequence.
struct Tile {
  int bh, q0;
  int nblk[2];   // key blocks each 128-row half attends to
  int n_iter;    // key blocks the tile loads (max of the two)
};

// Tile `idx` of the hand-out order.  Heads are taken in groups of `group_heads`; inside a group the
// index runs over the query tiles from the last (most key blocks under a causal mask) to the first,
// heads innermost.  About one group is in flight at a time, so its K/V (2*S*D elements per head)
// stays in L2 while the group's other query tiles read it.
__device__ __forceinline__ void decode_tile(const AttnArgs& a, int idx, Tile& t) {
  const int per_group = a.group_heads * a.n_qtiles;
  const int grp = idx / per_group, r = idx - grp * per_group;
  const int left = a.BH - grp * a.group_heads;
  const int hg = left < a.group_heads ? left : a.group_heads;
  t.q0 = (a.n_qtiles - 1 - r / hg) * BQ;
  t.bh = grp * a.group_heads + r % hg;
  const int kv_total = (a.S + BKV - 1) / BKV;
  t.n_iter = 0;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int row0 = t.q0 + h * BH_ROWS;
    int n;
    if (row0 >= a.S) n = 0;
    else if (a.causal) { const int lim = row0 / BKV + 1; n = lim < kv_total ? lim : kv_total; }
    else n = kv_total;
    t.nblk[h] = n;
    t.n_iter = n > t.n_iter ? n : t.n_iter;
  }
}

template <int HD, bool BF16>
__global__ void __launch_bounds__(ATT_THREADS, 1) attention_kernel(const __grid_constant__ AttnArgs a) {
  using L = AttnSmem<HD>;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + B_COUNT);
  volatile int* tile_ring = reinterpret_cast<volatile int*>(bars + B_COUNT + 1);   // TILE_SLOTS tile indices, -1 = no more

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#ifdef CDR_ATT_PROF
  volatile long long* prof_tab = reinterpret_cast<volatile long long*>(smem + L::PROF_OFF);
  for (int i = threadIdx.x; i < PROF_SLOTS; i += ATT_THREADS) prof_tab[i] = 0;
#endif

  if (warp == 0 && lane == 0) {
    sm100::prefetch_tensormap(&a.tmap_q);
    sm100::prefetch_tensormap(&a.tmap_k);
    sm100::prefetch_tensormap(&a.tmap_v);
    sm100::prefetch_tensormap(&a.tmap_o);
    for (int i = 0; i < B_COUNT; ++i) {
      const bool per_warp = (i >= B_PFULL && i < B_PFULL + 2) || (i >= B_OFREE && i < B_OFREE + 2);
      const bool slot_free = i >= B_TEMPTY && i < B_TEMPTY + TILE_SLOTS;
      // P and O-free: one arrival per softmax warp of the half; a tile slot is free once every reader has it
      sm100::mbar_init(&bars[i], slot_free ? TILE_READERS : per_warp ? 4 : 1);
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

  // one setmaxnreg per warp group, executed by all four of its warps
  if (warp < SOFTMAX_WARP0) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGS_CONTROL));
  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    // Runs ahead of the consumers across tile boundaries: the ring index never resets, and the Q
    // halves of the next tile are fetched as soon as the last S MMA of the current one is done.
    if (lane == 0) {
      int ring = 0;
      bool ok = true;
      // the first tile of a CTA is its block index; later ones come from the global counter, fetched
      // one tile ahead so that the atomic's latency hides behind the current tile's loads
      int idx = static_cast<int>(blockIdx.x);
      PROF_BEGIN(true);
      for (int k = 0; ok; ++k) {
        const int slot = k % TILE_SLOTS;
        PROF_ADD(true, 0);
        if (k >= TILE_SLOTS && !sm100::mbar_wait(&bars[B_TEMPTY + slot], (k / TILE_SLOTS - 1) & 1)) { sm100::report_timeout(a.status, 30); break; }
        PROF_ADD(true, 30);
        const bool valid = idx < a.total_tiles;
        tile_ring[slot] = valid ? idx : -1;
        sm100::mbar_arrive(&bars[B_TFULL + slot]);      // release: the index is visible to whoever sees the phase flip
        if (!valid) break;
        Tile t;
        decode_tile(a, idx, t);
        idx = static_cast<int>(gridDim.x + atomicAdd(a.next_tile, 1u));
        PROF_ADD(true, 0);
        if (k > 0 && !sm100::mbar_wait(&bars[B_QEMPTY], (k - 1) & 1)) { sm100::report_timeout(a.status, 21); break; }
        PROF_ADD(true, 21);
        PROF_COUNT(true, 1);
        const int active = (t.nblk[0] > 0) + (t.nblk[1] > 0);
        sm100::mbar_arrive_expect_tx(&bars[B_QFULL], active * L::TILE_BYTES);
        for (int h = 0; h < 2; ++h)
          if (t.nblk[h] > 0)
#pragma unroll
            for (int d = 0; d < HD / 64; ++d)
              sm100::tma_load_3d(smem + L::Q_OFF + h * L::TILE_BYTES + d * (128 * 128), &a.tmap_q, d * 64,
                                 t.q0 + h * BH_ROWS, t.bh, &bars[B_QFULL]);
        // ring tile i of the tile: K_j for i = 2j, V_j for i = 2j + 1
        for (int i = 0; i < 2 * t.n_iter; ++i) {
          const int r = ring + i, st = r % KV_STAGES, use = r / KV_STAGES;
          PROF_ADD(true, 0);
          if (use > 0 && !sm100::mbar_wait(&bars[B_EMPTY + st], (use - 1) & 1)) { sm100::report_timeout(a.status, 20); ok = false; break; }
          PROF_ADD(true, 20);
          sm100::mbar_arrive_expect_tx(&bars[B_FULL + st], L::TILE_BYTES);
          const void* tmap = (i & 1) ? static_cast<const void*>(&a.tmap_v) : static_cast<const void*>(&a.tmap_k);
#pragma unroll
          for (int d = 0; d < HD / 64; ++d)
            sm100::tma_load_3d(smem + L::KV_OFF + st * L::TILE_BYTES + d * (128 * 128), tmap, d * 64, (i >> 1) * BKV, t.bh,
                               &bars[B_FULL + st]);
        }
        ring += 2 * t.n_iter;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    // The whole warp runs this code convergently and one elected lane issues the tcgen05
    // instructions: with warp-uniform control flow the operand descriptors live in uniform
    // registers, where tcgen05.mma reads them, instead of being moved there before every
    // instruction (measured: ~95 cycles per MMA issued from a single-lane branch, more than the
    // 64 cycles a 128x128x16 MMA executes in).  Tiles follow one another without a gap: the first
    // scores of the next tile are issued right behind the last product of the current one, while
    // the softmax warps still write the current tile's output.
    {
      const bool leader = sm100::elect_one();
      constexpr uint32_t idesc_s = sm100::umma_idesc_f16(BH_ROWS, BKV, BF16, false, false);
      constexpr uint32_t idesc_o = sm100::umma_idesc_f16(BH_ROWS, HD, BF16, false, true);  // V is MN-major
      // every lane waits; the vote makes the outcome provably uniform
      PROF_BEGIN(leader);
      auto wait_all = [&](uint64_t* bar, uint32_t parity, int site) -> bool {
        PROF_ADD(leader, 2);                       // issue / bookkeeping time between waits
        const bool done = __all_sync(0xffffffffu, sm100::mbar_wait(bar, parity));
        PROF_ADD(leader, site);
        if (!done && leader) sm100::report_timeout(a.status, site);
        return done;
      };
      auto commit = [&](uint64_t* bar) {
        if (leader) sm100::umma_commit(bar);
        __syncwarp();
      };
      int ring = 0;                 // ring index of the current tile's K_0
      int blocks[2] = {0, 0};       // key blocks issued so far per half (phases of its S / P / PV barriers)
      int tiles_done[2] = {0, 0};   // tiles whose products are all issued, per half (gates the reuse of O_h)
      bool ok = true;

      for (int k = 0; ok; ++k) {
        const int slot = k % TILE_SLOTS;
        ok = wait_all(&bars[B_TFULL + slot], (k / TILE_SLOTS) & 1, 31);
        if (!ok) break;
        const int idx = tile_ring[slot];
        __syncwarp();
        if (leader) sm100::mbar_arrive(&bars[B_TEMPTY + slot]);
        if (idx < 0) break;
        Tile t;
        decode_tile(a, idx, t);
        const int n_iter = t.n_iter;
        ok = wait_all(&bars[B_QFULL], k & 1, 22);
        if (!ok) break;
        auto ring_wait = [&](int i, int site) { const int r = ring + i; return wait_all(&bars[B_FULL + r % KV_STAGES], (r / KV_STAGES) & 1, site); };
        auto ring_free = [&](int i) { commit(&bars[B_EMPTY + (ring + i) % KV_STAGES]); };
        // S_h(j) = Q_h K_j^T; the caller has already waited for K_j
        auto issue_s = [&](int h, int j) {
          const uint32_t q_addr = sm100::smem_u32(smem + L::Q_OFF + h * L::TILE_BYTES);
          const uint32_t k_addr = sm100::smem_u32(smem + L::KV_OFF + ((ring + 2 * j) % KV_STAGES) * L::TILE_BYTES);
          const uint32_t d = tmem_base + TMEM_S + h * 128;
          if (leader) {
#pragma unroll
            for (int kk = 0; kk < HD / 16; ++kk) {
              const uint32_t off = (kk / 4) * (128 * 128) + (kk % 4) * 32;
              sm100::umma_f16_ss(d, sm100::umma_desc_k_sw128(q_addr + off), sm100::umma_desc_k_sw128(k_addr + off), idesc_s,
                                 kk > 0 ? 1u : 0u);
            }
            sm100::umma_commit(&bars[B_SFULL + h]);
          }
          __syncwarp();
        };

        if (n_iter > 0) {
          ok = ring_wait(0, 23);
          if (!ok) break;
          sm100::tc_fence_after();
          for (int h = 0; h < 2; ++h)
            if (t.nblk[h] > 0) issue_s(h, 0);
          ring_free(0);                       // K_0 free once both S(0) are done
          if (n_iter == 1) commit(&bars[B_QEMPTY]);
        }
        for (int j = 0; j < n_iter && ok; ++j) {
          const bool next = j + 1 < n_iter;
          const int vt = 2 * j + 1, kt = 2 * j + 2;       // ring tiles of V_j and K_(j+1)
          ok = ring_wait(vt, 25);
          if (!ok) break;
          bool k_ready = false;
          const uint32_t v_addr = sm100::smem_u32(smem + L::KV_OFF + ((ring + vt) % KV_STAGES) * L::TILE_BYTES);
          for (int h = 0; h < 2 && ok; ++h) {
            if (j < t.nblk[h]) {
              // the first product of a tile overwrites O_h: the previous tile's epilogue must have read it
              if (j == 0 && tiles_done[h] > 0) {
                ok = wait_all(&bars[B_OFREE + h], (tiles_done[h] - 1) & 1, 28);
                if (!ok) break;
              }
              ok = wait_all(&bars[B_PFULL + h], blocks[h] & 1, 26 + h);     // sites 26 and 27 (timeouts); also cycle-accounting slots
              if (!ok) break;
              ++blocks[h];
              sm100::tc_fence_after();
              const uint32_t p_tmem = tmem_base + TMEM_S + h * 128;   // packed bf16 pairs: 8 columns per 16 keys
              if (leader) {
#pragma unroll
                for (int kk = 0; kk < BKV / 16; ++kk) {
                  const uint64_t vdesc = sm100::umma_desc_mn_sw128(v_addr + kk * (16 * 128), 128 * 128);
                  sm100::umma_f16_ts(tmem_base + TMEM_O + h * 128, p_tmem + kk * 8, vdesc, idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
                }
                sm100::umma_commit(&bars[B_PVDONE + h]);
              }
              __syncwarp();
              if (j == t.nblk[h] - 1) ++tiles_done[h];
            }
            if (next && j + 1 < t.nblk[h]) {
              if (!k_ready) {
                ok = ring_wait(kt, 24);
                if (!ok) break;
                k_ready = true;
                sm100::tc_fence_after();
              }
              issue_s(h, j + 1);
            }
          }
          if (!ok) break;
          ring_free(vt);
          if (next) ring_free(kt);
          if (j + 2 == n_iter) commit(&bars[B_QEMPTY]);   // every S of this tile is issued: Q may be replaced
        }
        ring += 2 * n_iter;
      }
    }
  } else if (warp >= SOFTMAX_WARP0) {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(REGS_SOFTMAX));
    // ------------------------------------------------------------ softmax / correction / epilogue
    const int g = (warp - SOFTMAX_WARP0) >> 2;       // half this warp group serves
    const int q = warp & 3;              // TMEM lane quadrant
    const int row_in_half = q * 32 + lane;
    const uint32_t lane_sel = static_cast<uint32_t>(q * 32) << 16;
    const uint32_t s_taddr = tmem_base + TMEM_S + g * 128 + lane_sel;
    const uint32_t o_taddr = tmem_base + TMEM_O + g * 128 + lane_sel;
    int n = 0;                           // key blocks consumed so far over all tiles (barrier phases)
    bool ok = true;
#ifdef CDR_ATT_PROF
    const bool pw = q == 0 && lane == 0;   // one accounting thread per half
    const int pb = 64 + 32 * g;
#endif
    PROF_BEGIN(pw);

    for (int k = 0; ok; ++k) {
      const int slot = k % TILE_SLOTS;
      PROF_ADD(pw, pb + 0);
      if (!sm100::mbar_wait(&bars[B_TFULL + slot], (k / TILE_SLOTS) & 1)) { sm100::report_timeout(a.status, 32); break; }
      PROF_ADD(pw, pb + 1);
      const int idx = tile_ring[slot];
      __syncwarp();
      if (lane == 0) sm100::mbar_arrive(&bars[B_TEMPTY + slot]);
      if (idx < 0) break;
      Tile t;
      decode_tile(a, idx, t);
      const int n_my = t.nblk[g];
      if (n_my == 0) continue;
      const int row0 = t.q0 + g * BH_ROWS;
      const int row = row0 + row_in_half;
      float m_ref = -INFINITY, l0 = 0.0f, l1 = 0.0f;

      for (int j = 0; j < n_my; ++j, ++n) {
        PROF_ADD(pw, pb + 0);
        if (!sm100::mbar_wait(&bars[B_SFULL + g], n & 1)) { sm100::report_timeout(a.status, 33); ok = false; break; }
        PROF_ADD(pw, pb + 2);
        PROF_COUNT(pw, pb + 10);
        sm100::tc_fence_after();
        uint32_t sr[4][32];
#pragma unroll
        for (int c = 0; c < 4; ++c) sm100::tmem_ld32(s_taddr + c * 32, sr[c]);
        sm100::tmem_ld_wait();
        PROF_ADD(pw, pb + 3);

        const int key0 = j * BKV;
        const bool need_mask = (a.causal && key0 + BKV - 1 > row0) || (key0 + BKV > a.S);
        if (need_mask) {
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int key = key0 + c * 32 + i;
              if (key >= a.S || (a.causal && key > row)) sr[c][i] = __float_as_uint(-INFINITY);   // exp2(-inf) is exactly 0
            }
        }

        if (j == 0) {
          // first block of a tile: the reference maximum is this block's own
          float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // four independent chains of 3-input max
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int i = 0; i < 16; ++i)
              mx[i & 3] = max3(mx[i & 3], __uint_as_float(sr[c][2 * i]), __uint_as_float(sr[c][2 * i + 1]));
          m_ref = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * a.scale_log2;  // scale > 0: max commutes with the scaling
          const float neg_m = (m_ref == -INFINITY) ? 0.0f : -m_ref;
          store_p<BF16, CDR_ATT_EMU, false>(sr, a.scale_log2, neg_m, l0, l1, s_taddr);
          PROF_ADD(pw, pb + 4);
        } else {
          // later blocks: P against the reference maximum already held, the block's own maximum on the
          // side.  S_h(j) was issued after P_h(j-1) V_(j-1), and MMAs complete in order: O_h is stable here.
          float l0s = l0, l1s = l1;
          const float neg_m = (m_ref == -INFINITY) ? 0.0f : -m_ref;
          const float bmax = store_p<BF16, CDR_ATT_EMU, true>(sr, a.scale_log2, neg_m, l0s, l1s, s_taddr) * a.scale_log2;
          PROF_ADD(pw, pb + 5);
          if (__any_sync(0xffffffffu, bmax > m_ref + kRescaleThreshold)) {
            PROF_COUNT(pw, pb + 11);
            // rare: the block's maximum outgrew the reference; rescale the accumulator and redo P
            const float m_new = fmaxf(m_ref, bmax);
            const float alpha = (m_ref == -INFINITY) ? 0.0f : fast_exp2(m_ref - m_new);
            l0 *= alpha;
            l1 *= alpha;
            m_ref = m_new;
#pragma unroll 1
            for (int c = 0; c < HD / 32; ++c) {
              uint32_t o[32];
              sm100::tmem_ld32(o_taddr + c * 32, o);
              sm100::tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
              sm100::tmem_st32(o_taddr + c * 32, o);
            }
            sm100::tmem_st_wait();      // the first P of this block must be in place before it is overwritten
            const float neg_m2 = (m_ref == -INFINITY) ? 0.0f : -m_ref;
            store_p<BF16, CDR_ATT_EMU, false>(sr, a.scale_log2, neg_m2, l0, l1, s_taddr);
            PROF_ADD(pw, pb + 6);
          } else {
            l0 = l0s;
            l1 = l1s;
          }
        }
        sm100::tmem_st_wait();
        sm100::tc_fence_before();
        __syncwarp();
        if (lane == 0) sm100::mbar_arrive(&bars[B_PFULL + g]);
        PROF_ADD(pw, pb + 7);
      }
      if (!ok) break;
      PROF_ADD(pw, pb + 0);

      // ---- epilogue: O / l, rounded to the output type; O_h is handed back after the last read
      if (!sm100::mbar_wait(&bars[B_PVDONE + g], (n - 1) & 1)) { sm100::report_timeout(a.status, 29); ok = false; break; }
      PROF_ADD(pw, pb + 8);
      sm100::tc_fence_after();
      const float inv = 1.0f / (l0 + l1);
      // Each warp packs 32 columns of its 32 rows into its shared-memory stage and hands them to the TMA
      // unit (one tiled store per chunk, issued by lane 0): the global stores leave the softmax warps'
      // path, and rows beyond S are clipped by the tensor map.
      unsigned char* stage = smem + L::STAGE_OFF + (warp - SOFTMAX_WARP0) * (32 * 64);
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t o[32];
        sm100::tmem_ld32(o_taddr + c * 32, o);
        sm100::tmem_ld_wait();
        if (c == HD / 32 - 1) {
          sm100::tc_fence_before();
          __syncwarp();
          if (lane == 0) sm100::mbar_arrive(&bars[B_OFREE + g]);
        }
        uint32_t w[16];
#pragma unroll
        for (int tt = 0; tt < 16; ++tt)
          w[tt] = pack_pair<BF16>(__uint_as_float(o[tt * 2]) * inv, __uint_as_float(o[tt * 2 + 1]) * inv);
        if (lane == 0) sm100::bulk_wait_read<0>();      // the previous store has read the stage
        __syncwarp();
#pragma unroll
        for (int gq = 0; gq < 4; ++gq)
          *reinterpret_cast<uint4*>(stage + lane * 64 + gq * 16) = make_uint4(w[gq * 4], w[gq * 4 + 1], w[gq * 4 + 2], w[gq * 4 + 3]);
        sm100::fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          sm100::tma_store_3d(&a.tmap_o, stage, c * 32, row0 + q * 32, t.bh);
          sm100::bulk_commit();
        }
      }
      PROF_ADD(pw, pb + 9);
    }
    if (lane == 0) sm100::bulk_wait<0>();     // every output store of this warp has completed
  }

  sm100::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    sm100::tc_fence_after();
    sm100::tmem_dealloc(tmem_base, ATT_TMEM_COLS);
  }
#ifdef CDR_ATT_PROF
  {
    long long* dst = reinterpret_cast<long long*>(reinterpret_cast<unsigned char*>(a.next_tile) + 256) + static_cast<size_t>(blockIdx.x) * PROF_SLOTS;
    for (int i = threadIdx.x; i < PROF_SLOTS; i += ATT_THREADS) dst[i] = prof_tab[i];
  }
#endif
}

}  // namespace
// ---------------------------------------------------------------- host side
int attention_workspace(const cdr_tensor*, int, size_t* bytes) {
  // O, the running max and the running sum never leave TMEM / registers; the scratch is the
  // counter the CTAs take their next tile from (cleared by every launch)
  *bytes = 256 + static_cast<size_t>(PROF_SLOTS) * 8 * 1024;   // the accounting table exists in development builds only
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
    // setmaxnreg.inc waits until the CTA's register pool (threads x registers per thread at launch)
    // can cover the request; if the compiled kernel ever got fewer registers than the split below
    // assumes, that wait would never end -- refuse to launch instead
    cudaFuncAttributes fa;
    CDR_CUDA_TRY(cudaFuncGetAttributes(&fa, kern));
    if (fa.numRegs * ATT_THREADS < 128 * REGS_CONTROL + (ATT_THREADS - 128) * REGS_SOFTMAX) {
      set_error("attention: kernel was built with %d registers per thread, the register split needs %d", fa.numRegs,
                (128 * REGS_CONTROL + (ATT_THREADS - 128) * REGS_SOFTMAX + ATT_THREADS - 1) / ATT_THREADS);
      return CDR_ERR_UNSUPPORTED;
    }
    CDR_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    configured_dev[dev & 63] = true;
  }
  const int64_t tiles = static_cast<int64_t>(a.BH) * a.n_qtiles;
  if (tiles > 0x3fffffff) { set_error("attention: too many tiles"); return CDR_ERR_UNSUPPORTED; }
  const int64_t sms = sm_count();
  const int64_t grid = tiles < sms ? tiles : sms;   // persistent: one CTA per SM walks its share of the tiles
  kern<<<static_cast<unsigned>(grid), ATT_THREADS, smem, stream>>>(a);
  CDR_CUDA_TRY(cudaGetLastError());
  return CDR_OK;
}
}  // namespace

int launch_attention(const cdr_tensor* ins, int n_in, const cdr_tensor* outs, int n_out, const cdr_attn_params* p,
                     void* ws, size_t ws_bytes, cudaStream_t stream) {
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

  if (!ws || ws_bytes < sizeof(unsigned int)) {
    set_error("attention: workspace of %zu bytes required, got %zu", (size_t)256, ws ? ws_bytes : (size_t)0);
    return CDR_ERR_WORKSPACE;
  }
  if (reinterpret_cast<uintptr_t>(ws) & 3u) { set_error("attention: workspace must be 4-byte aligned"); return CDR_ERR_MISALIGNED; }

  AttnArgs a;
  const int bf16 = q.dtype == CDR_BF16;
  if (int rc = make_tensor_map_3d(&a.tmap_q, ins[0].data, bf16, D, S, BH, 64, 128)) return rc;
  if (int rc = make_tensor_map_3d(&a.tmap_k, ins[1].data, bf16, D, S, BH, 64, 128)) return rc;
  if (int rc = make_tensor_map_3d(&a.tmap_v, ins[2].data, bf16, D, S, BH, 64, 128)) return rc;
  if (int rc = make_tensor_map_3d_plain(&a.tmap_o, out.data, bf16, D, S, BH, 32, 32)) return rc;
  a.out = out.data;
  a.S = static_cast<int>(S);
  a.BH = static_cast<int>(BH);
  a.n_qtiles = static_cast<int>((S + BQ - 1) / BQ);
  if (BH * ((S + BQ - 1) / BQ) > 0x3fffffff) { set_error("attention: too many tiles"); return CDR_ERR_UNSUPPORTED; }
  a.total_tiles = a.BH * a.n_qtiles;
  // heads per scheduling group: the CTAs in flight cover about one group's tiles
  a.group_heads = sm_count() / a.n_qtiles;
  if (a.group_heads < 1) a.group_heads = 1;
  if (a.group_heads > a.BH) a.group_heads = a.BH;
  a.next_tile = static_cast<unsigned int*>(ws);
  CDR_CUDA_TRY(cudaMemsetAsync(a.next_tile, 0, sizeof(unsigned int), stream));
  a.scale_log2 = p->scale * 1.4426950408889634f;
  a.causal = p->causal ? 1 : 0;
  a.status = device_status_ptr();
  if (D == 128) return bf16 ? launch_attention_cfg<128, true>(a, stream) : launch_attention_cfg<128, false>(a, stream);
  return bf16 ? launch_attention_cfg<64, true>(a, stream) : launch_attention_cfg<64, false>(a, stream);
}

}  // namespace cdr
