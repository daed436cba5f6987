// K2 -- elementwise chain + reduction epilogue.
//
// The reference only sketches reductions as comment templates
// (conductor/codegen/operator_registry.py:399-458) and clusters "elementwise
// producers feeding a reduction" in conductor/optimization/fusion.py:714-728; the
// executed arithmetic is eager `mean(relu(x*w+b), dim=-1, dtype=float32)`
// (examples/reduce_mean_fusion_example.py:52-102).
//
// HBM-bound: the full-size inputs are read once (128-bit streaming loads), the
// row-broadcast operands (w, b) are loaded once per CTA and kept in registers for
// every row the CTA handles, the chain's intermediates never leave registers, and
// only one value per row is written.  Row sums use warp shuffles plus one
// shared-memory hop between the warps of a CTA.
//
// bf16 chains are evaluated with packed bf16x2 mul/add/max (each correctly rounded,
// never fused), which is bit-identical to eager's "fp32 op, round to bf16" and keeps
// the instruction count low enough to stay memory-bound.
#include <type_traits>

#include <stdlib.h>

#include "cdr_common.cuh"

namespace cdr {

int validate_ew_program(const cdr_ew_params* p, int n_in, int n_out);
int launch_full_reduce_jit(const void* const* in, void* out, float* partials, unsigned int* ticket, const int* in_dt,
                           int out_dt, const cdr_ew_params& p, int reduce_op, int64_t n_units, int64_t cols, int E,
                           int grid, cudaStream_t stream);
int launch_row_reduce_jit(const void* const* in, void* out, const int* in_dt, int out_dt, const cdr_ew_params& p,
                          int reduce_op, int64_t rows, int64_t cols, int E, cudaStream_t stream);
int64_t expected_input_numel(int mode, int64_t n, int64_t cols);

namespace {

// ---------------------------------------------------------------- packed chains
// A "word" is 32 bits of a 16-byte vector: one fp32 or two bf16.
// apply(): adds the chain value(s) of the word to the accumulator.
struct WordIdentityF32 {
  using elem = float;
  static constexpr int NROW = 0;
  __device__ __forceinline__ static void apply(uint32_t x, const uint32_t*, float& acc) {
    acc += __uint_as_float(x);
  }
};
struct WordMulAddReluF32 {
  using elem = float;
  static constexpr int NROW = 2;
  __device__ __forceinline__ static void apply(uint32_t x, const uint32_t* row, float& acc) {
    float v = __fadd_rn(__fmul_rn(__uint_as_float(x), __uint_as_float(row[0])), __uint_as_float(row[1]));
    v = v > 0.0f ? v : (v != v ? v : 0.0f);
    acc += v;
  }
};
__device__ __forceinline__ void acc_bf16x2(uint32_t w, float& acc) {
  acc += __uint_as_float(w << 16);
  acc += __uint_as_float(w & 0xffff0000u);
}
struct WordIdentityBF16 {
  using elem = __nv_bfloat16;
  static constexpr int NROW = 0;
  __device__ __forceinline__ static void apply(uint32_t x, const uint32_t*, float& acc) { acc_bf16x2(x, acc); }
};
struct WordMulAddReluBF16 {
  using elem = __nv_bfloat16;
  static constexpr int NROW = 2;
  __device__ __forceinline__ static void apply(uint32_t x, const uint32_t* row, float& acc) {
    const __nv_bfloat162 xv = *reinterpret_cast<const __nv_bfloat162*>(&x);
    const __nv_bfloat162 wv = *reinterpret_cast<const __nv_bfloat162*>(&row[0]);
    const __nv_bfloat162 bv = *reinterpret_cast<const __nv_bfloat162*>(&row[1]);
    const __nv_bfloat162 zero = __float2bfloat162_rn(0.0f);
    __nv_bfloat162 v = __hmax2_nan(__hadd2_rn(__hmul2_rn(xv, wv), bv), zero);
    acc_bf16x2(*reinterpret_cast<uint32_t*>(&v), acc);
  }
};

struct RowArgs {
  const void* full;      // the one full-size input, [rows, cols]
  const void* row[2];    // row-broadcast inputs, [cols]
  void* out;             // [rows]
  int32_t out_dtype;
  int32_t mean;          // 1: divide the sum by cols
  int64_t rows;
  int64_t cols;
};

__device__ __forceinline__ void store_result(void* out, int dt, int64_t i, float v) {
  if (dt == CDR_F32) static_cast<float*>(out)[i] = v;
  else if (dt == CDR_BF16) static_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn(v);
  else static_cast<__half*>(out)[i] = __float2half_rn(v);
}

// NT threads per CTA; a thread owns vectors {t, t+NT, ...} (VPT of them) of every row;
// the CTA walks row blocks of RB rows, grid-stride.  EXACT: cols == NT*VPT*V, rows % RB == 0
// and the tensor has fewer than 2^31 elements, so the hot loop carries no bounds predicates
// and indexes with 32-bit arithmetic (measured 22.5 us against 25.7 us for the guarded form on
// the bf16 [16384, 4096] benchmark shape; a pure read of the same bytes takes 20.8 us).
// A shared-memory ring filled by bulk (TMA) copies was measured too and lost (27-29 us): the
// consumer side, not bytes in flight, limits this kernel.
template <class Chain, int NT, int VPT, int RB, bool EXACT>
__global__ void __launch_bounds__(NT, (768 / NT > 0 ? 768 / NT : 1)) row_reduce_named_kernel(const __grid_constant__ RowArgs a) {
  using T = typename Chain::elem;
  using idx_t = typename std::conditional<EXACT, int32_t, int64_t>::type;
  constexpr int V = 16 / sizeof(T);
  constexpr int NW = NT / 32;
  constexpr int NROW = Chain::NROW;
  __shared__ float part[2][RB][NW];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const idx_t cols = static_cast<idx_t>(a.cols), rows = static_cast<idx_t>(a.rows);
  const idx_t vec_per_row = cols / V;

  // Programmatic dependent launch: let the next kernel of the stream be scheduled while this one
  // runs, and wait for the previous one to finish (and flush) before the first global access.
  // Both are no-ops when the launch does not carry the attribute.
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");

  // row-broadcast operands: loaded once, register resident for the whole kernel
  uint4 rowv[NROW > 0 ? NROW : 1][VPT];
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const idx_t v = tid + j * NT;
#pragma unroll
    for (int r = 0; r < NROW; ++r)
      rowv[r][j] = (EXACT || v < vec_per_row) ? ld_cached16(static_cast<const T*>(a.row[r]) + v * V)
                                              : make_uint4(0, 0, 0, 0);
  }

  const idx_t n_blocks = (rows + RB - 1) / RB;
  int parity = 0;
  for (idx_t blk = blockIdx.x; blk < n_blocks; blk += gridDim.x, parity ^= 1) {
    const idx_t row0 = blk * RB;
    const T* base = static_cast<const T*>(a.full) + row0 * cols + tid * V;
    uint4 x[RB][VPT];
#pragma unroll
    for (int r = 0; r < RB; ++r) {
#pragma unroll
      for (int j = 0; j < VPT; ++j) {
        const bool live = EXACT || (row0 + r < rows && tid + j * NT < vec_per_row);
        x[r][j] = live ? ld_stream16(base + r * cols + j * (NT * V)) : make_uint4(0, 0, 0, 0);
      }
    }
    float acc[RB];
#pragma unroll
    for (int r = 0; r < RB; ++r) {
      float a0 = 0.0f, a1 = 0.0f;
#pragma unroll
      for (int j = 0; j < VPT; ++j) {
        if (EXACT || tid + j * NT < vec_per_row) {  // a padded vector would add chain(0) != 0
          uint32_t rw[4][NROW > 0 ? NROW : 1];
#pragma unroll
          for (int q = 0; q < NROW; ++q) {
            rw[0][q] = rowv[q][j].x; rw[1][q] = rowv[q][j].y; rw[2][q] = rowv[q][j].z; rw[3][q] = rowv[q][j].w;
          }
          Chain::apply(x[r][j].x, rw[0], a0);
          Chain::apply(x[r][j].y, rw[1], a1);
          Chain::apply(x[r][j].z, rw[2], a0);
          Chain::apply(x[r][j].w, rw[3], a1);
        }
      }
      acc[r] = warp_sum(a0 + a1);
    }
    if (NW == 1) {
      if (lane == 0) {
#pragma unroll
        for (int r = 0; r < RB; ++r)
          if (EXACT || row0 + r < rows) {
            const float s = a.mean ? __fdiv_rn(acc[r], static_cast<float>(a.cols)) : acc[r];
            store_result(a.out, a.out_dtype, row0 + r, s);
          }
      }
    } else {
      if (lane == 0) {
#pragma unroll
        for (int r = 0; r < RB; ++r) part[parity][r][warp] = acc[r];
      }
      __syncthreads();
      if (tid < RB && (EXACT || row0 + tid < rows)) {
        float s = 0.0f;
#pragma unroll
        for (int w = 0; w < NW; ++w) s += part[parity][tid][w];
        if (a.mean) s = __fdiv_rn(s, static_cast<float>(a.cols));
        store_result(a.out, a.out_dtype, row0 + tid, s);
      }
    }
  }
}

// ---------------------------------------------------------------- generic path
constexpr int kMaxRegs = CDR_EW_MAX_INPUTS + CDR_EW_MAX_INSTR;

struct GenArgs {
  const void* in[CDR_EW_MAX_INPUTS];
  int32_t in_dtype[CDR_EW_MAX_INPUTS];
  void* out;
  int32_t out_dtype;
  int32_t reduce_op;
  int64_t rows;
  int64_t cols;
  cdr_ew_params prog;
};

__device__ __forceinline__ float gen_load(const void* base, int dt, int64_t i) {
  switch (dt) {
    case CDR_F32: return static_cast<const float*>(base)[i];
    case CDR_BF16: return __bfloat162float(static_cast<const __nv_bfloat16*>(base)[i]);
    case CDR_F16: return __half2float(static_cast<const __half*>(base)[i]);
    default: return 0.0f;
  }
}

__device__ __forceinline__ float gen_op(int op, float a, float b, float c, float imm) {
  switch (op) {
    case CDR_OP_ADD: return __fadd_rn(a, b);
    case CDR_OP_SUB: return __fsub_rn(a, b);
    case CDR_OP_MUL: return __fmul_rn(a, b);
    case CDR_OP_DIV: return __fdiv_rn(a, b);
    case CDR_OP_RELU: return a > 0.0f ? a : (a != a ? a : 0.0f);
    case CDR_OP_NEG: return -a;
    case CDR_OP_ABS: return fabsf(a);
    case CDR_OP_EXP: return expf(a);
    case CDR_OP_LOG: return logf(a);
    case CDR_OP_SQRT: return __fsqrt_rn(a);
    case CDR_OP_SIGMOID: return __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-a)));
    case CDR_OP_TANH: return tanhf(a);
    case CDR_OP_SIN: return sinf(a);
    case CDR_OP_COS: return cosf(a);
    case CDR_OP_MAX: return (a != a || b != b) ? (a + b) : fmaxf(a, b);
    case CDR_OP_MIN: return (a != a || b != b) ? (a + b) : fminf(a, b);
    case CDR_OP_ADDCDIV: return __fadd_rn(a, __fdiv_rn(__fmul_rn(imm, b), c));
    case CDR_OP_ADDCMUL: return __fadd_rn(a, __fmul_rn(__fmul_rn(imm, b), c));
    case CDR_OP_CONST: return imm;
    case CDR_OP_COPY: return a;
    case CDR_OP_ADD_IMM: return __fadd_rn(a, imm);
    case CDR_OP_MUL_IMM: return __fmul_rn(a, imm);
    case CDR_OP_RSUB_IMM: return __fsub_rn(imm, a);
    case CDR_OP_RDIV_IMM: return __fdiv_rn(imm, a);
    case CDR_OP_GT: return a > b ? 1.0f : 0.0f;
    case CDR_OP_GE: return a >= b ? 1.0f : 0.0f;
    case CDR_OP_LT: return a < b ? 1.0f : 0.0f;
    case CDR_OP_LE: return a <= b ? 1.0f : 0.0f;
    case CDR_OP_EQ: return a == b ? 1.0f : 0.0f;
    case CDR_OP_NE: return a != b ? 1.0f : 0.0f;
    case CDR_OP_WHERE: return a != 0.0f ? b : c;
    case CDR_OP_RSQRT: return __fdiv_rn(1.0f, __fsqrt_rn(a));
    case CDR_OP_SILU: return __fdiv_rn(a, __fadd_rn(1.0f, expf(-a)));
    case CDR_OP_GELU: return __fmul_rn(__fmul_rn(a, 0.5f), __fadd_rn(1.0f, erff(__fmul_rn(a, 0.70710678118654752440f))));
    case CDR_OP_ERF: return erff(a);
    default: return 0.0f;
  }
}

// Chain value of flat element `i` of the [rows, cols] view.
__device__ __forceinline__ float gen_eval(const GenArgs& a, int64_t i, int64_t row, int64_t col) {
  float reg[kMaxRegs];
  const cdr_ew_params& p = a.prog;
  for (int k = 0; k < p.n_inputs; ++k) {
    const int m = p.input_mode[k];
    const int64_t idx = m == CDR_IN_FULL ? i : m == CDR_IN_ROW ? col : m == CDR_IN_COL ? row : 0;
    reg[k] = gen_load(a.in[k], a.in_dtype[k], idx);
  }
  for (int k = 0; k < p.n_instr; ++k) {
    const cdr_ew_instr ins = p.instr[k];
    reg[p.n_inputs + k] = round_to_dtype(gen_op(ins.op, reg[ins.a], reg[ins.b], reg[ins.c], ins.imm), ins.round_to);
  }
  return reg[p.out_reg[0]];
}

__device__ __forceinline__ float red_identity(int op) {
  return op == CDR_RED_MAX ? -INFINITY : op == CDR_RED_MIN ? INFINITY : 0.0f;
}
__device__ __forceinline__ float red_combine(int op, float a, float b) {
  if (op == CDR_RED_MAX) return (a != a || b != b) ? (a + b) : fmaxf(a, b);
  if (op == CDR_RED_MIN) return (a != a || b != b) ? (a + b) : fminf(a, b);
  return a + b;
}
__device__ __forceinline__ float warp_combine(int op, float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = red_combine(op, v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
template <int NT>
__device__ __forceinline__ float cta_combine(int op, float v, float* smem) {
  v = warp_combine(op, v);
  if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = red_identity(op);
  if (threadIdx.x < 32) {
    if (threadIdx.x < NT / 32) r = smem[threadIdx.x];
    r = warp_combine(op, r);
  }
  __syncthreads();
  return r;  // valid in warp 0
}

// One CTA per row (grid-stride over rows), scalar interpreter.
template <int NT>
__global__ void __launch_bounds__(NT) row_reduce_generic_kernel(const __grid_constant__ GenArgs a) {
  __shared__ float smem[NT / 32];
  for (int64_t row = blockIdx.x; row < a.rows; row += gridDim.x) {
    float acc = red_identity(a.reduce_op);
    for (int64_t c = threadIdx.x; c < a.cols; c += NT)
      acc = red_combine(a.reduce_op, acc, gen_eval(a, row * a.cols + c, row, c));
    const float r = cta_combine<NT>(a.reduce_op, acc, smem);
    if (threadIdx.x == 0) {
      const float v = a.reduce_op == CDR_RED_MEAN ? __fdiv_rn(r, static_cast<float>(a.cols)) : r;
      store_result(a.out, a.out_dtype, row, v);
    }
  }
}

// Full reduction, stage 1+2 in one launch: every CTA writes one partial into scratch,
// the CTA that finishes last (ticket counter in scratch) folds the partials.
struct FullArgs {
  GenArgs g;          // rows*cols = all elements
  float* partials;    // scratch: one float per CTA
  unsigned int* ticket;  // scratch: zero before the launch
};

template <int NT>
__global__ void __launch_bounds__(NT) full_reduce_kernel(const __grid_constant__ FullArgs a) {
  __shared__ float smem[NT / 32];
  __shared__ bool is_last;
  const int64_t n = a.g.rows * a.g.cols;
  const int op = a.g.reduce_op;
  float acc = red_identity(op);
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * NT + threadIdx.x; i < n; i += static_cast<int64_t>(gridDim.x) * NT)
    acc = red_combine(op, acc, gen_eval(a.g, i, i / a.g.cols, i % a.g.cols));
  float r = cta_combine<NT>(op, acc, smem);
  if (threadIdx.x == 0) {
    a.partials[blockIdx.x] = r;
    __threadfence();
    const unsigned int t = atomicAdd(a.ticket, 1u);
    is_last = (t == gridDim.x - 1);
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  acc = red_identity(op);
  for (int i = threadIdx.x; i < static_cast<int>(gridDim.x); i += NT)
    acc = red_combine(op, acc, __ldcg(a.partials + i));
  r = cta_combine<NT>(op, acc, smem);
  if (threadIdx.x == 0) {
    const float v = op == CDR_RED_MEAN ? __fdiv_rn(r, static_cast<float>(n)) : r;
    store_result(a.g.out, a.g.out_dtype, 0, v);
    *a.ticket = 0;  // leave the counter ready for the next launch
  }
}

// ---------------------------------------------------------------- host side
enum RowChain { kRNone = 0, kRIdentity, kRMulAddRelu };

RowChain match_row_chain(const cdr_ew_params& p, int dt, int* full_idx, int* row_idx) {
  if (p.n_inputs == 1 && p.n_instr == 0 && p.out_reg[0] == 0 && p.input_mode[0] == CDR_IN_FULL) {
    *full_idx = 0;
    return kRIdentity;
  }
  if (p.n_inputs == 3 && p.n_instr == 3 && p.out_reg[0] == 5) {
    for (int k = 0; k < 3; ++k)
      if (p.instr[k].round_to != dt) return kRNone;
    const cdr_ew_instr &m = p.instr[0], &s = p.instr[1], &r = p.instr[2];
    if (m.op != CDR_OP_MUL || s.op != CDR_OP_ADD || r.op != CDR_OP_RELU || r.a != 4) return kRNone;
    // mul(x, w) with x full and w row; add(mul, b) with b row (either operand order)
    int x = -1, w = -1, b = -1;
    if (p.input_mode[m.a] == CDR_IN_FULL && p.input_mode[m.b] == CDR_IN_ROW) { x = m.a; w = m.b; }
    else if (p.input_mode[m.b] == CDR_IN_FULL && p.input_mode[m.a] == CDR_IN_ROW) { x = m.b; w = m.a; }
    else return kRNone;
    if (m.a >= 3 || m.b >= 3) return kRNone;
    if (s.a == 3 && s.b < 3) b = s.b; else if (s.b == 3 && s.a < 3) b = s.a; else return kRNone;
    if (b == x || b == w || p.input_mode[b] != CDR_IN_ROW) return kRNone;
    *full_idx = x; row_idx[0] = w; row_idx[1] = b;
    return kRMulAddRelu;
  }
  return kRNone;
}

inline bool pdl_enabled() {
  static const bool on = getenv("CDR_DISABLE_PDL") == nullptr;
  return on;
}

template <class Chain, int NT, int VPT, int RB, bool EXACT>
int launch_named_variant(const RowArgs& a, cudaStream_t s) {
  auto kern = row_reduce_named_kernel<Chain, NT, VPT, RB, EXACT>;
  // the occupancy query costs microseconds of host time: ask once per kernel instance
  static int cached_per_sm = 0;
  if (cached_per_sm == 0) {
    int q = 0;
    CDR_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&q, kern, NT, 0));
    cached_per_sm = q < 1 ? 1 : q;
  }
  int per_sm = cached_per_sm;
  // 768 resident threads per SM measured best (3 CTAs of 256: 22.6 us; 4: 23.1; 6: 24.6)
  if (per_sm > 768 / NT && NT <= 768) per_sm = 768 / NT;
  const int64_t n_blocks = (a.rows + RB - 1) / RB;
  int64_t grid = static_cast<int64_t>(sm_count()) * per_sm;
  if (grid > n_blocks) grid = n_blocks;
  // every CTA gets the same number of row blocks: a last, sparsely populated round would run
  // latency-bound and cost as much as a full one
  int64_t rounds = (n_blocks + grid - 1) / grid;
  // a short problem (two or three rounds of row blocks) runs faster as ONE round of more CTAs: every
  // CTA then issues all of its loads at once instead of paying a second trip to memory after the first
  // (2048 rows of the bf16 [16384, 4096] benchmark shape: 4.90 -> 4.55 us)
  if (rounds > 1 && rounds <= 3 && n_blocks <= static_cast<int64_t>(sm_count()) * (2048 / NT)) rounds = 1;
  grid = (n_blocks + rounds - 1) / rounds;
  // launched with programmatic stream serialization: the kernel begins with griddepcontrol.wait,
  // so it may be scheduled before its predecessor in the stream has drained
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid));
  cfg.blockDim = dim3(NT);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  CDR_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, a));
  return CDR_OK;
}

template <class Chain, int NT, int VPT>
int launch_named_cfg(const RowArgs& a, cudaStream_t s) {
  constexpr int RB = (VPT >= 8) ? 1 : (8 / VPT);  // 8 16-byte loads in flight per thread
  constexpr int V = 16 / sizeof(typename Chain::elem);
  const bool exact = a.cols == static_cast<int64_t>(NT) * VPT * V && a.rows % RB == 0 &&
                     a.rows * a.cols < (int64_t{1} << 31);
  if (exact) return launch_named_variant<Chain, NT, VPT, RB, true>(a, s);
  return launch_named_variant<Chain, NT, VPT, RB, false>(a, s);
}

template <class Chain>
int launch_named_row(const RowArgs& a, cudaStream_t s) {
  constexpr int V = 16 / sizeof(typename Chain::elem);
  const int64_t vec = a.cols / V;
  if (vec <= 32) return launch_named_cfg<Chain, 32, 1>(a, s);
  if (vec <= 64) return launch_named_cfg<Chain, 64, 1>(a, s);
  if (vec <= 128) return launch_named_cfg<Chain, 128, 1>(a, s);
  if (vec <= 256) return launch_named_cfg<Chain, 256, 1>(a, s);
  if (vec <= 512) return launch_named_cfg<Chain, 256, 2>(a, s);
  if (vec <= 1024) return launch_named_cfg<Chain, 256, 4>(a, s);
  if (vec <= 2048) return launch_named_cfg<Chain, 256, 8>(a, s);
  return CDR_ERR_UNSUPPORTED;
}

int check_reduce_inputs(const cdr_tensor* ins, int n_in, const cdr_reduce_params* p, int64_t rows, int64_t cols,
                        const char* who) {
  for (int i = 0; i < n_in; ++i) {
    if (!ins[i].data) { set_error("%s: input %d has a null pointer", who, i); return CDR_ERR_BAD_ARG; }
    if (!is_contiguous(ins[i])) { set_error("%s: input %d is not contiguous", who, i); return CDR_ERR_BAD_ARG; }
    if (ins[i].dtype != CDR_F32 && ins[i].dtype != CDR_BF16 && ins[i].dtype != CDR_F16) {
      set_error("%s: input %d has dtype %d; only floating types reduce", who, i, ins[i].dtype);
      return CDR_ERR_UNSUPPORTED;
    }
    const int64_t want = expected_input_numel(p->chain.input_mode[i], rows * cols, cols);
    if (numel(ins[i]) != want) {
      set_error("%s: input %d has %lld elements, expected %lld", who, i, (long long)numel(ins[i]), (long long)want);
      return CDR_ERR_BAD_ARG;
    }
  }
  if (p->reduce_op < CDR_RED_SUM || p->reduce_op > CDR_RED_MIN) {
    set_error("%s: unknown reduce op %d", who, p->reduce_op);
    return CDR_ERR_BAD_ARG;
  }
  return CDR_OK;
}

void fill_gen_args(GenArgs& g, const cdr_tensor* ins, int n_in, const cdr_tensor& out, const cdr_reduce_params* p,
                   int64_t rows, int64_t cols) {
  for (int i = 0; i < n_in; ++i) { g.in[i] = ins[i].data; g.in_dtype[i] = ins[i].dtype; }
  g.out = out.data; g.out_dtype = out.dtype; g.reduce_op = p->reduce_op;
  g.rows = rows; g.cols = cols; g.prog = p->chain;
}

}  // namespace

int launch_row_reduce(const cdr_tensor* ins, int n_in, const cdr_tensor* outs, int n_out,
                      const cdr_reduce_params* p, cudaStream_t stream) {
  if (!p) { set_error("row_reduce: params is null"); return CDR_ERR_BAD_ARG; }
  if (int rc = validate_ew_program(&p->chain, n_in, n_out)) return rc;
  if (n_out != 1 || n_in < 1) { set_error("row_reduce: needs >=1 input and exactly one output"); return CDR_ERR_BAD_ARG; }
  // the [rows, cols] view comes from the first full-size input
  int full = -1;
  for (int i = 0; i < n_in; ++i)
    if (p->chain.input_mode[i] == CDR_IN_FULL) { full = i; break; }
  if (full < 0) { set_error("row_reduce: no full-size input"); return CDR_ERR_BAD_ARG; }
  const cdr_tensor& x = ins[full];
  if (x.rank < 1) { set_error("row_reduce: input rank 0"); return CDR_ERR_BAD_ARG; }
  const int64_t cols = x.shape[x.rank - 1];
  const int64_t rows = cols ? numel(x) / cols : 0;
  const cdr_tensor& out = outs[0];
  if (numel(out) != rows || !is_contiguous(out)) {
    set_error("row_reduce: output must be contiguous with %lld elements", (long long)rows);
    return CDR_ERR_BAD_ARG;
  }
  if (out.dtype != CDR_F32 && out.dtype != CDR_BF16 && out.dtype != CDR_F16) {
    set_error("row_reduce: output dtype %d unsupported", out.dtype);
    return CDR_ERR_UNSUPPORTED;
  }
  if (int rc = check_reduce_inputs(ins, n_in, p, rows, cols, "row_reduce")) return rc;
  if (rows == 0) return CDR_OK;
  if (!out.data) { set_error("row_reduce: output pointer is null"); return CDR_ERR_BAD_ARG; }
  if (cols == 0) { set_error("row_reduce: reduction over an empty dimension"); return CDR_ERR_UNSUPPORTED; }

  // named fast path: sum/mean, one dtype, aligned, whole vectors per row
  const int dt = x.dtype;
  bool same = true;
  for (int i = 0; i < n_in; ++i) same &= ins[i].dtype == dt && aligned16(ins[i].data);
  const int V = 16 / dtype_size(dt);
  if (same && (dt == CDR_F32 || dt == CDR_BF16) && cols % V == 0 &&
      (p->reduce_op == CDR_RED_SUM || p->reduce_op == CDR_RED_MEAN)) {
    int fidx = 0, ridx[2] = {0, 0};
    const RowChain c = match_row_chain(p->chain, dt, &fidx, ridx);
    if (c != kRNone) {
      RowArgs a{};
      a.full = ins[fidx].data; a.row[0] = ins[ridx[0]].data; a.row[1] = ins[ridx[1]].data;
      a.out = out.data; a.out_dtype = out.dtype; a.mean = p->reduce_op == CDR_RED_MEAN;
      a.rows = rows; a.cols = cols;
      int rc = CDR_ERR_UNSUPPORTED;
      if (c == kRIdentity && dt == CDR_F32) rc = launch_named_row<WordIdentityF32>(a, stream);
      else if (c == kRIdentity && dt == CDR_BF16) rc = launch_named_row<WordIdentityBF16>(a, stream);
      else if (c == kRMulAddRelu && dt == CDR_F32) rc = launch_named_row<WordMulAddReluF32>(a, stream);
      else if (c == kRMulAddRelu && dt == CDR_BF16) rc = launch_named_row<WordMulAddReluBF16>(a, stream);
      if (rc != CDR_ERR_UNSUPPORTED) return rc;
    }
  }

  GenArgs g{};
  fill_gen_args(g, ins, n_in, out, p, rows, cols);

  // no ahead-of-time instance: instantiate the vector skeleton for this program at run time
  {
    bool any16 = false, ok = true;
    for (int i = 0; i < n_in; ++i) any16 |= dtype_size(ins[i].dtype) == 2;
    const int E = any16 ? 8 : 4;
    for (int i = 0; i < n_in; ++i) {
      const int m = p->chain.input_mode[i];
      if (m == CDR_IN_FULL || m == CDR_IN_ROW) ok &= aligned16(ins[i].data);
    }
    if (ok && cols % E == 0) {
      const int rc = launch_row_reduce_jit(g.in, g.out, g.in_dtype, g.out_dtype, p->chain, p->reduce_op, rows, cols, E, stream);
      if (rc != CDR_ERR_UNSUPPORTED) return rc;
    }
  }

  int64_t grid = rows;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  if (grid > cap) grid = cap;
  row_reduce_generic_kernel<256><<<static_cast<unsigned>(grid), 256, 0, stream>>>(g);
  CDR_CUDA_TRY(cudaGetLastError());
  return CDR_OK;
}

// scratch layout of the full reduction: [ticket: 256 B][partials: one float per CTA]
static int full_reduce_grid() { return sm_count() * 4; }

int full_reduce_workspace(const cdr_tensor*, int, size_t* bytes) {
  *bytes = 256 + sizeof(float) * static_cast<size_t>(full_reduce_grid());
  return CDR_OK;
}

int launch_full_reduce(const cdr_tensor* ins, int n_in, const cdr_tensor* outs, int n_out,
                       const cdr_reduce_params* p, void* ws, size_t ws_bytes, cudaStream_t stream,
                       bool allow_runtime_instance) {
  if (!p) { set_error("full_reduce: params is null"); return CDR_ERR_BAD_ARG; }
  if (int rc = validate_ew_program(&p->chain, n_in, n_out)) return rc;
  if (n_out != 1 || n_in < 1) { set_error("full_reduce: needs >=1 input and exactly one output"); return CDR_ERR_BAD_ARG; }
  int full = -1;
  for (int i = 0; i < n_in; ++i)
    if (p->chain.input_mode[i] == CDR_IN_FULL) { full = i; break; }
  if (full < 0) { set_error("full_reduce: no full-size input"); return CDR_ERR_BAD_ARG; }
  const cdr_tensor& x = ins[full];
  const int64_t cols = x.rank > 0 ? x.shape[x.rank - 1] : 1;
  const int64_t n = numel(x);
  const int64_t rows = cols ? n / cols : 0;
  if (numel(outs[0]) != 1 || !outs[0].data) { set_error("full_reduce: output must hold one element"); return CDR_ERR_BAD_ARG; }
  if (outs[0].dtype != CDR_F32 && outs[0].dtype != CDR_BF16 && outs[0].dtype != CDR_F16) {
    set_error("full_reduce: output dtype %d unsupported", outs[0].dtype);
    return CDR_ERR_UNSUPPORTED;
  }
  if (int rc = check_reduce_inputs(ins, n_in, p, rows, cols, "full_reduce")) return rc;
  if (n == 0) { set_error("full_reduce: reduction over an empty tensor"); return CDR_ERR_UNSUPPORTED; }
  size_t need = 0;
  full_reduce_workspace(ins, n_in, &need);
  if (!ws || ws_bytes < need) {
    set_error("full_reduce: workspace of %zu bytes required, got %zu", need, ws ? ws_bytes : (size_t)0);
    return CDR_ERR_WORKSPACE;
  }
  if (reinterpret_cast<uintptr_t>(ws) & 255u) { set_error("full_reduce: workspace must be 256-byte aligned"); return CDR_ERR_MISALIGNED; }
  FullArgs a{};
  fill_gen_args(a.g, ins, n_in, outs[0], p, rows, cols);
  a.ticket = static_cast<unsigned int*>(ws);
  a.partials = reinterpret_cast<float*>(static_cast<char*>(ws) + 256);
  int64_t grid = (n + 255) / 256;
  if (grid > full_reduce_grid()) grid = full_reduce_grid();
  CDR_CUDA_TRY(cudaMemsetAsync(a.ticket, 0, sizeof(unsigned int), stream));
  // vector-shaped problems get a run-time instance of the streaming skeleton (its first use
  // compiles and loads a module, which allocates: callers that must not allocate skip it)
  if (allow_runtime_instance) {
    bool any16 = false, ok = true;
    for (int i = 0; i < n_in; ++i) any16 |= dtype_size(ins[i].dtype) == 2;
    const int E = any16 ? 8 : 4;
    for (int i = 0; i < n_in; ++i) {
      const int m = p->chain.input_mode[i];
      if (m == CDR_IN_FULL || m == CDR_IN_ROW) ok &= aligned16(ins[i].data);
      if (m == CDR_IN_ROW || m == CDR_IN_COL) ok &= cols % E == 0;
    }
    if (ok && n % E == 0) {
      int64_t jgrid = (n / E + 255) / 256;
      if (jgrid > full_reduce_grid()) jgrid = full_reduce_grid();
      const int rc = launch_full_reduce_jit(a.g.in, a.g.out, a.partials, a.ticket, a.g.in_dtype, a.g.out_dtype, p->chain,
                                            p->reduce_op, n / E, cols, E, static_cast<int>(jgrid), stream);
      if (rc != CDR_ERR_UNSUPPORTED) return rc;
    }
  }
  full_reduce_kernel<256><<<static_cast<unsigned>(grid), 256, 0, stream>>>(a);
  CDR_CUDA_TRY(cudaGetLastError());
  return CDR_OK;
}


// ---------------------------------------------------------------- column sums: out[n] = sum_m x[m, n]
// HBM-bound (every element read once).  The [M, N] matrix is cut into strips of 256 columns (a
// warp reads 32 x 16 bytes of a row: whole 512-byte lines) and chunks of rows; a CTA of 8 warps
// sums its chunk of its strip in fp32 registers, folds the warps through shared memory and
// writes one partial row to scratch.  The last CTA of a strip to finish (a ticket per strip) adds
// the chunk partials in chunk order -- a fixed order, so the result is the same on every run --
// and rounds to the output type.  Columns past the last whole vector take a scalar path.
namespace {

constexpr int CS_STRIP = 256, CS_WARPS = 8;

struct ColSumArgs {
  const void* x;
  void* out;
  float* partials;         // [chunks][N]
  unsigned int* tickets;   // [strips]
  int64_t M, N;
  int chunks, rows_per_chunk;
  int dtype;
};

template <typename T>
__device__ __forceinline__ float cs_load(const T* p) { return static_cast<float>(*p); }
template <>
__device__ __forceinline__ float cs_load<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <>
__device__ __forceinline__ float cs_load<__half>(const __half* p) { return __half2float(*p); }

template <typename T>
__global__ void __launch_bounds__(CS_WARPS * 32) col_sum_kernel(const ColSumArgs a) {
  constexpr int V = 16 / sizeof(T);                 // elements per 16-byte vector
  constexpr int PER_LANE = CS_STRIP / 32;            // 8 columns per lane
  constexpr int VECS = PER_LANE / V;                 // 1 vector (16-bit types) or 2 (fp32)
  __shared__ float fold[CS_WARPS][CS_STRIP];
  __shared__ unsigned int last_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int strip = blockIdx.x, chunk = blockIdx.y;
  const int64_t col0 = static_cast<int64_t>(strip) * CS_STRIP + lane * PER_LANE;
  const int64_t r0 = static_cast<int64_t>(chunk) * a.rows_per_chunk;
  int64_t r1 = r0 + a.rows_per_chunk;
  if (r1 > a.M) r1 = a.M;
  const T* x = static_cast<const T*>(a.x);
  float acc[PER_LANE];
#pragma unroll
  for (int i = 0; i < PER_LANE; ++i) acc[i] = 0.0f;
  const bool vec = (a.N % V) == 0 && (reinterpret_cast<uintptr_t>(a.x) & 15u) == 0 && col0 + PER_LANE <= a.N;
  if (vec) {
#pragma unroll 4
    for (int64_t r = r0 + warp; r < r1; r += CS_WARPS) {
      const uint4* p = reinterpret_cast<const uint4*>(x + r * a.N + col0);
#pragma unroll
      for (int v = 0; v < VECS; ++v) {
        const uint4 q = __ldcs(p + v);
        const T* e = reinterpret_cast<const T*>(&q);
#pragma unroll
        for (int i = 0; i < V; ++i) acc[v * V + i] += cs_load<T>(e + i);
      }
    }
  } else {
    for (int64_t r = r0 + warp; r < r1; r += CS_WARPS)
#pragma unroll
      for (int i = 0; i < PER_LANE; ++i)
        if (col0 + i < a.N) acc[i] += cs_load<T>(x + r * a.N + col0 + i);
  }
#pragma unroll
  for (int i = 0; i < PER_LANE; ++i) fold[warp][lane * PER_LANE + i] = acc[i];
  __syncthreads();
  // one thread per column of the strip: the CTA's partial, warps added in index order
  const int c = threadIdx.x;
  const int64_t col = static_cast<int64_t>(strip) * CS_STRIP + c;
  if (col < a.N) {
    float s = 0.0f;
#pragma unroll
    for (int w = 0; w < CS_WARPS; ++w) s += fold[w][c];
    a.partials[static_cast<int64_t>(chunk) * a.N + col] = s;
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) last_flag = atomicAdd(&a.tickets[strip], 1u) == static_cast<unsigned int>(a.chunks - 1);
  __syncthreads();
  if (!last_flag) return;
  __threadfence();
  if (col < a.N) {
    float s = 0.0f;
    for (int k = 0; k < a.chunks; ++k) s += __ldcg(&a.partials[static_cast<int64_t>(k) * a.N + col]);
    if (a.dtype == CDR_F32) static_cast<float*>(a.out)[col] = s;
    else if (a.dtype == CDR_BF16) static_cast<__nv_bfloat16*>(a.out)[col] = __float2bfloat16_rn(s);
    else static_cast<__half*>(a.out)[col] = __float2half_rn(s);
  }
}

// strips x chunks CTAs: enough chunks to fill the device about four times over, at least 32 rows each
void col_sum_geometry(int64_t M, int64_t N, int* strips, int* chunks, int* rows_per_chunk) {
  *strips = static_cast<int>((N + CS_STRIP - 1) / CS_STRIP);
  int64_t want = (static_cast<int64_t>(sm_count()) * 4 + *strips - 1) / *strips;
  const int64_t most = (M + 31) / 32;
  if (want > most) want = most;
  if (want < 1) want = 1;
  if (want > 1024) want = 1024;
  *rows_per_chunk = static_cast<int>((M + want - 1) / want);
  *chunks = static_cast<int>((M + *rows_per_chunk - 1) / *rows_per_chunk);
}

int col_sum_shape(const cdr_tensor* ins, int n_in, const cdr_tensor* outs, int n_out, int64_t* M, int64_t* N) {
  if (n_in != 1 || n_out != 1) { set_error("col_sum: expects one input and one output"); return CDR_ERR_BAD_ARG; }
  *N = numel(outs[0]);
  const int64_t n = numel(ins[0]);
  if (*N <= 0 || n % *N != 0) { set_error("col_sum: the input's element count must be a multiple of the output's"); return CDR_ERR_BAD_ARG; }
  *M = n / *N;
  return CDR_OK;
}

}  // namespace

int col_sum_workspace(const cdr_tensor* ins, int n_in, const cdr_tensor* outs, int n_out, size_t* bytes) {
  int64_t M = 0, N = 0;
  if (int rc = col_sum_shape(ins, n_in, outs, n_out, &M, &N)) return rc;
  int strips, chunks, rpc;
  col_sum_geometry(M > 0 ? M : 1, N, &strips, &chunks, &rpc);
  // [tickets: strips words, rounded up to 256 bytes][partials: chunks x N floats]
  *bytes = ((static_cast<size_t>(strips) * 4 + 255) & ~static_cast<size_t>(255)) + static_cast<size_t>(chunks) * N * sizeof(float);
  return CDR_OK;
}

int launch_col_sum(const cdr_tensor* ins, int n_in, const cdr_tensor* outs, int n_out, void* ws, size_t ws_bytes,
                   cudaStream_t stream) {
  int64_t M = 0, N = 0;
  if (int rc = col_sum_shape(ins, n_in, outs, n_out, &M, &N)) return rc;
  const cdr_tensor &x = ins[0], &out = outs[0];
  if (!is_contiguous(x) || !is_contiguous(out)) { set_error("col_sum: tensors must be contiguous"); return CDR_ERR_BAD_ARG; }
  if (x.dtype != out.dtype || (x.dtype != CDR_F32 && x.dtype != CDR_BF16 && x.dtype != CDR_F16)) {
    set_error("col_sum: input and output must share one floating dtype");
    return CDR_ERR_UNSUPPORTED;
  }
  if (!out.data || (M > 0 && !x.data)) { set_error("col_sum: null pointer"); return CDR_ERR_BAD_ARG; }
  size_t need = 0;
  col_sum_workspace(ins, n_in, outs, n_out, &need);
  if (!ws || ws_bytes < need) { set_error("col_sum: workspace of %zu bytes required, got %zu", need, ws ? ws_bytes : (size_t)0); return CDR_ERR_WORKSPACE; }
  if (reinterpret_cast<uintptr_t>(ws) & 255u) { set_error("col_sum: workspace must be 256-byte aligned"); return CDR_ERR_MISALIGNED; }
  if (M == 0) {   // an empty sum is zero
    CDR_CUDA_TRY(cudaMemsetAsync(out.data, 0, static_cast<size_t>(N) * dtype_size(out.dtype), stream));
    return CDR_OK;
  }
  ColSumArgs a{};
  int strips;
  col_sum_geometry(M, N, &strips, &a.chunks, &a.rows_per_chunk);
  const size_t ticket_bytes = (static_cast<size_t>(strips) * 4 + 255) & ~static_cast<size_t>(255);
  a.x = x.data; a.out = out.data; a.M = M; a.N = N; a.dtype = x.dtype;
  a.tickets = static_cast<unsigned int*>(ws);
  a.partials = reinterpret_cast<float*>(static_cast<char*>(ws) + ticket_bytes);
  CDR_CUDA_TRY(cudaMemsetAsync(a.tickets, 0, static_cast<size_t>(strips) * 4, stream));
  const dim3 grid(static_cast<unsigned>(strips), static_cast<unsigned>(a.chunks));
  if (x.dtype == CDR_F32) col_sum_kernel<float><<<grid, CS_WARPS * 32, 0, stream>>>(a);
  else if (x.dtype == CDR_BF16) col_sum_kernel<__nv_bfloat16><<<grid, CS_WARPS * 32, 0, stream>>>(a);
  else col_sum_kernel<__half><<<grid, CS_WARPS * 32, 0, stream>>>(a);
  CDR_CUDA_TRY(cudaGetLastError());
  return CDR_OK;
}

}  // namespace cdr

// =====================================================================================
// cdr_full_reduce_noalloc: the full reduction for callers that must not allocate.
//
// Some hosts cannot call cudaMalloc on the hot path: an inference server or another
// framework's memory pool that reserved all of HBM at start-up (so a driver allocation would
// fail, or is forbidden by the host's policy), and latency-critical loops that cannot absorb
// the device-wide synchronisation an allocation implies.  For them the scratch the full
// reduction needs (one ticket counter plus one fp32 partial per CTA) lives in a fixed array
// inside this library's device image instead of in a caller-provided workspace.
//
//  * Capacity: kStaticPartials partial sums, i.e. kStaticScratchBytes = 256 + 4*1024 = 4352
//    bytes, held by every GPU that loads the library until the process exits.  The reduction
//    uses 4 CTAs per SM, so this covers devices with up to 256 SMs; a launch that would need
//    more slots is rejected with CDR_ERR_UNSUPPORTED and a message naming both numbers.
//  * The first call on a device looks up the array's device address (cudaGetSymbolAddress)
//    and caches it; make that first call before starting any stream capture.
//  * All calls on a device share the array.  The ticket is cleared at the start of every
//    call; partials are overwritten.  Two calls whose kernels overlap on the GPU (different
//    streams, no ordering between them) race on it: serialise them.
//  * No cudaMalloc, cudaFree or allocating library call happens in here.  In particular the
//    call never takes the run-time-instance path of the ordinary entry point (whose first use
//    per program compiles with NVRTC and loads a module into device memory): it always runs the
//    kernel that was compiled into this library.
// =====================================================================================
namespace cdr {
namespace {

constexpr int kStaticPartials = 1024;
constexpr size_t kStaticScratchBytes = 256 + sizeof(float) * kStaticPartials;

// In host code this name is only a handle for cudaGetSymbolAddress, never a device pointer.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

void* g_static_scratch_ptr[64] = {nullptr};

// Device address of the scratch array on the current device (looked up once per device).
int static_scratch_address(void** out) {
  int dev = 0;
  CDR_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) { set_error("full_reduce_noalloc: device %d out of range", dev); return CDR_ERR_BAD_ARG; }
  if (!g_static_scratch_ptr[dev]) {
    void* p = nullptr;
    CDR_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_scratch));
    g_static_scratch_ptr[dev] = p;
  }
  *out = g_static_scratch_ptr[dev];
  return CDR_OK;
}

}  // namespace
}  // namespace cdr

extern "C" CDR_API int cdr_full_reduce_noalloc(const cdr_tensor* inputs, int n_inputs, const cdr_tensor* outputs,
                                               int n_outputs, const void* params, size_t params_bytes,
                                               void* cuda_stream) {
  using namespace cdr;
  clear_error();
  if (int rc = check_lists(inputs, n_inputs, outputs, n_outputs)) return rc;
  if (!params || params_bytes != sizeof(cdr_reduce_params)) {
    set_error("full_reduce_noalloc: expects a %zu-byte cdr_reduce_params block", sizeof(cdr_reduce_params));
    return CDR_ERR_BAD_ARG;
  }
  size_t need = 0;
  full_reduce_workspace(inputs, n_inputs, &need);
  if (need > kStaticScratchBytes) {
    set_error("full_reduce_noalloc: this device needs %zu bytes of scratch (%zu partial sums), the built-in array "
              "holds %zu bytes (%d partial sums); use cdr_launch with a caller workspace instead",
              need, (need - 256) / sizeof(float), kStaticScratchBytes, kStaticPartials);
    return CDR_ERR_UNSUPPORTED;
  }
  void* scratch = nullptr;
  if (int rc = static_scratch_address(&scratch)) return rc;
  return launch_full_reduce(inputs, n_inputs, outputs, n_outputs, static_cast<const cdr_reduce_params*>(params),
                            scratch, kStaticScratchBytes, static_cast<cudaStream_t>(cuda_stream),
                            /*allow_runtime_instance=*/false);
}
