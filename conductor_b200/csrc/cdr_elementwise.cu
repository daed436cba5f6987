// K1 -- elementwise-chain template.
//
// One launch evaluates a whole fused elementwise cluster (the reference emits such a
// cluster as one `foreach` body: conductor/codegen/dslgen.py:524-737; the scalar
// definition of the flagship chain is samples/fused/mul_add.co:19-21, of addcdiv
// choreo-op/addcdiv-dynamic.co:412-416, of relu
// choreo-op/activation-relu-fp32-templated-kernel.co:11-18).
//
// HBM-bound: every external input is read once and every output written once with
// 128-bit coalesced accesses; intermediates (LOCAL buffers) live in registers.
// Arithmetic is done op by op in fp32 with round-to-nearest and NO fma contraction,
// and each op's result is rounded to the op's dtype, so results equal eager execution
// of the same graph bit for bit for +,-,*,/ and relu.
//
// Two instantiation routes:
//   * named chains (mul_add, addcdiv, relu, add, sub, mul, div, mul_add_relu):
//     the chain is a compile-time functor, fully in registers;
//   * any other program: a register-file interpreter (uniform control flow, the
//     register file lives in local memory), float or integer.
#include "cdr_common.cuh"

namespace cdr {

int launch_elementwise_jit(const void* const* in, void* const* out, const int* in_dt, const int* out_dt,
                           const cdr_ew_params& p, int64_t n_units, int64_t cols, int E, cudaStream_t stream);

namespace {

constexpr int kThreads = 256;

struct EwArgs {
  const void* in[CDR_EW_MAX_INPUTS];
  void* out[CDR_EW_MAX_OUTPUTS];
  int32_t in_dtype[CDR_EW_MAX_INPUTS];
  int32_t out_dtype[CDR_EW_MAX_OUTPUTS];
  int64_t n;     // elements of the output
  int64_t cols;  // innermost extent of the [rows, cols] view used for broadcasts
  int64_t first; // first element this launch handles (scalar tail launches)
  cdr_ew_params prog;
};

// ---------------------------------------------------------------- op semantics
__device__ __forceinline__ float relu_f(float x) { return x > 0.0f ? x : (x != x ? x : 0.0f); }

__device__ __forceinline__ float apply_op_f(int op, float a, float b, float c, float imm) {
  switch (op) {
    case CDR_OP_ADD: return __fadd_rn(a, b);
    case CDR_OP_SUB: return __fsub_rn(a, b);
    case CDR_OP_MUL: return __fmul_rn(a, b);
    case CDR_OP_DIV: return __fdiv_rn(a, b);
    case CDR_OP_RELU: return relu_f(a);
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

// Integer registers are 64-bit two's complement; storing to int32 truncates, which is
// exactly int32 wrap-around for + - * (bit-exact against eager integer tensors).
__device__ __forceinline__ int64_t apply_op_i(int op, int64_t a, int64_t b, int64_t c, float imm) {
  const int64_t k = static_cast<int64_t>(imm);
  switch (op) {
    case CDR_OP_ADD: return static_cast<int64_t>(static_cast<uint64_t>(a) + static_cast<uint64_t>(b));
    case CDR_OP_SUB: return static_cast<int64_t>(static_cast<uint64_t>(a) - static_cast<uint64_t>(b));
    case CDR_OP_MUL: return static_cast<int64_t>(static_cast<uint64_t>(a) * static_cast<uint64_t>(b));
    case CDR_OP_RELU: return a > 0 ? a : 0;
    case CDR_OP_NEG: return static_cast<int64_t>(0ull - static_cast<uint64_t>(a));
    case CDR_OP_ABS: return a < 0 ? static_cast<int64_t>(0ull - static_cast<uint64_t>(a)) : a;
    case CDR_OP_MAX: return a > b ? a : b;
    case CDR_OP_MIN: return a < b ? a : b;
    case CDR_OP_ADDCMUL:
      return static_cast<int64_t>(static_cast<uint64_t>(a) +
                                  static_cast<uint64_t>(k) * static_cast<uint64_t>(b) * static_cast<uint64_t>(c));
    case CDR_OP_CONST: return k;
    case CDR_OP_COPY: return a;
    case CDR_OP_ADD_IMM: return static_cast<int64_t>(static_cast<uint64_t>(a) + static_cast<uint64_t>(k));
    case CDR_OP_MUL_IMM: return static_cast<int64_t>(static_cast<uint64_t>(a) * static_cast<uint64_t>(k));
    case CDR_OP_RSUB_IMM: return static_cast<int64_t>(static_cast<uint64_t>(k) - static_cast<uint64_t>(a));
    case CDR_OP_GT: return a > b;
    case CDR_OP_GE: return a >= b;
    case CDR_OP_LT: return a < b;
    case CDR_OP_LE: return a <= b;
    case CDR_OP_EQ: return a == b;
    case CDR_OP_NE: return a != b;
    case CDR_OP_WHERE: return a != 0 ? b : c;
    default: return 0;
  }
}

// ---------------------------------------------------------------- named chains
// Each functor: NIN inputs, apply() returns the single output.  T is the dtype every
// op of the chain is rounded to.
template <typename T> struct ChainMulAdd {
  static constexpr int NIN = 3;
  __device__ __forceinline__ static float apply(const float* r) {
    return round_as<T>(__fadd_rn(round_as<T>(__fmul_rn(r[0], r[1])), r[2]));
  }
};
template <typename T> struct ChainMulAddRelu {
  static constexpr int NIN = 3;
  __device__ __forceinline__ static float apply(const float* r) {
    return relu_f(round_as<T>(__fadd_rn(round_as<T>(__fmul_rn(r[0], r[1])), r[2])));
  }
};
template <typename T> struct ChainAddCDiv1 {  // addcdiv with value == 1 (addcdiv-dynamic.co:412-416)
  static constexpr int NIN = 3;
  __device__ __forceinline__ static float apply(const float* r) {
    return round_as<T>(__fadd_rn(r[0], __fdiv_rn(r[1], r[2])));
  }
};
template <typename T> struct ChainRelu {
  static constexpr int NIN = 1;
  __device__ __forceinline__ static float apply(const float* r) { return relu_f(r[0]); }
};
template <typename T, int OP> struct ChainBinary {
  static constexpr int NIN = 2;
  __device__ __forceinline__ static float apply(const float* r) {
    return round_as<T>(apply_op_f(OP, r[0], r[1], 0.0f, 0.0f));
  }
};

// ---------------------------------------------------------------- input access
// Load E consecutive output-aligned elements of one input as fp32.
template <typename T, int E>
__device__ __forceinline__ void load_unit(const void* base, int mode, int64_t elem0, int64_t cols,
                                          float* f) {
  constexpr int V = Pack16<T>::N;
  const T* p = static_cast<const T*>(base);
  if (mode == CDR_IN_FULL) {
#pragma unroll
    for (int k = 0; k < E / V; ++k) Pack16<T>::unpack(ld_stream16(p + elem0 + k * V), f + k * V);
  } else if (mode == CDR_IN_ROW) {
    const int64_t c = elem0 % cols;  // E divides cols on this path: no row straddling
#pragma unroll
    for (int k = 0; k < E / V; ++k) Pack16<T>::unpack(ld_cached16(p + c + k * V), f + k * V);
  } else {
    const int64_t idx = (mode == CDR_IN_COL) ? (elem0 / cols) : 0;
    const float v = to_f32<T>(p[idx]);
#pragma unroll
    for (int k = 0; k < E; ++k) f[k] = v;
  }
}

template <typename T, int E>
__device__ __forceinline__ void store_unit(void* base, int64_t elem0, const float* f) {
  constexpr int V = Pack16<T>::N;
  T* p = static_cast<T*>(base);
#pragma unroll
  for (int k = 0; k < E / V; ++k) st_stream16(p + elem0 + k * V, Pack16<T>::pack(f + k * V));
}

__device__ __forceinline__ float load_scalar_f(const void* base, int dt, int64_t i) {
  switch (dt) {
    case CDR_F32: return static_cast<const float*>(base)[i];
    case CDR_BF16: return __bfloat162float(static_cast<const __nv_bfloat16*>(base)[i]);
    case CDR_F16: return __half2float(static_cast<const __half*>(base)[i]);
    case CDR_I32: return static_cast<float>(static_cast<const int32_t*>(base)[i]);
    case CDR_I64: return static_cast<float>(static_cast<const int64_t*>(base)[i]);
    case CDR_BOOL: return static_cast<const uint8_t*>(base)[i] ? 1.0f : 0.0f;
    default: return 0.0f;
  }
}
__device__ __forceinline__ void store_scalar_f(void* base, int dt, int64_t i, float v) {
  switch (dt) {
    case CDR_F32: static_cast<float*>(base)[i] = v; break;
    case CDR_BF16: static_cast<__nv_bfloat16*>(base)[i] = __float2bfloat16_rn(v); break;
    case CDR_F16: static_cast<__half*>(base)[i] = __float2half_rn(v); break;
    case CDR_BOOL: static_cast<uint8_t*>(base)[i] = v != 0.0f; break;
    case CDR_I32: static_cast<int32_t*>(base)[i] = static_cast<int32_t>(v); break;
    case CDR_I64: static_cast<int64_t*>(base)[i] = static_cast<int64_t>(v); break;
    default: break;
  }
}
__device__ __forceinline__ int64_t load_scalar_i(const void* base, int dt, int64_t i) {
  switch (dt) {
    case CDR_I32: return static_cast<const int32_t*>(base)[i];
    case CDR_I64: return static_cast<const int64_t*>(base)[i];
    case CDR_BOOL: return static_cast<const uint8_t*>(base)[i] ? 1 : 0;
    default: return 0;
  }
}
__device__ __forceinline__ void store_scalar_i(void* base, int dt, int64_t i, int64_t v) {
  switch (dt) {
    case CDR_I32: static_cast<int32_t*>(base)[i] = static_cast<int32_t>(v); break;
    case CDR_I64: static_cast<int64_t*>(base)[i] = v; break;
    case CDR_BOOL: static_cast<uint8_t*>(base)[i] = v != 0; break;
    default: break;
  }
}

__device__ __forceinline__ int64_t input_index(int mode, int64_t i, int64_t cols) {
  switch (mode) {
    case CDR_IN_FULL: return i;
    case CDR_IN_ROW: return i % cols;
    case CDR_IN_COL: return i / cols;
    default: return 0;
  }
}

// ---------------------------------------------------------------- kernels
// Named chain, vector path.  Each CTA covers kThreads*UNROLL units of E elements;
// all loads of a thread are issued before the first use (UNROLL*NIN*E/V 16-byte
// requests in flight per thread).  UNROLL is 4 for 32-bit types and 1 for 16-bit types, whose
// units unpack to twice the registers (bf16 mul_add: 4.2 TB/s with two units, 6.1 with one).
// ALLFULL drops the per-input broadcast-mode switch when no input is broadcast.
template <class Chain, typename T, typename TO, int UNROLL, bool ALLFULL>
__global__ void __launch_bounds__(kThreads) ew_named_kernel(const __grid_constant__ EwArgs a) {
  constexpr int VI = Pack16<T>::N, VO = Pack16<TO>::N;
  constexpr int E = VI > VO ? VI : VO;
  constexpr int NIN = Chain::NIN;
  const int64_t n_units = a.n / E;
  const int64_t unit0 = static_cast<int64_t>(blockIdx.x) * (kThreads * UNROLL) + threadIdx.x;

  float r[UNROLL][NIN][E];
#pragma unroll
  for (int u = 0; u < UNROLL; ++u) {
    const int64_t unit = unit0 + static_cast<int64_t>(u) * kThreads;
    if (unit < n_units) {
#pragma unroll
      for (int i = 0; i < NIN; ++i)
        load_unit<T, E>(a.in[i], ALLFULL ? CDR_IN_FULL : a.prog.input_mode[i], unit * E, a.cols, r[u][i]);
    }
  }
#pragma unroll
  for (int u = 0; u < UNROLL; ++u) {
    const int64_t unit = unit0 + static_cast<int64_t>(u) * kThreads;
    if (unit < n_units) {
      float o[E];
#pragma unroll
      for (int e = 0; e < E; ++e) {
        float in[NIN];
#pragma unroll
        for (int i = 0; i < NIN; ++i) in[i] = r[u][i][e];
        o[e] = Chain::apply(in);
      }
      store_unit<TO, E>(a.out[0], unit * E, o);
    }
  }
}

// Interpreter over a float register file, E elements per thread-iteration.
constexpr int kMaxRegs = CDR_EW_MAX_INPUTS + CDR_EW_MAX_INSTR;

template <int E>
__device__ __forceinline__ void interpret_f(const cdr_ew_params& p, float (*reg)[E]) {
  for (int k = 0; k < p.n_instr; ++k) {
    const cdr_ew_instr ins = p.instr[k];
#pragma unroll
    for (int e = 0; e < E; ++e) {
      const float v = apply_op_f(ins.op, reg[ins.a][e], reg[ins.b][e], reg[ins.c][e], ins.imm);
      reg[p.n_inputs + k][e] = round_to_dtype(v, ins.round_to);
    }
  }
}

template <typename T, typename TO>
__global__ void __launch_bounds__(kThreads) ew_interp_vec_kernel(const __grid_constant__ EwArgs a) {
  constexpr int VI = Pack16<T>::N, VO = Pack16<TO>::N;
  constexpr int E = VI > VO ? VI : VO;
  const int64_t n_units = a.n / E;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  float reg[kMaxRegs][E];
  for (int64_t unit = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; unit < n_units;
       unit += stride) {
    for (int i = 0; i < a.prog.n_inputs; ++i)
      load_unit<T, E>(a.in[i], a.prog.input_mode[i], unit * E, a.cols, reg[i]);
    interpret_f<E>(a.prog, reg);
    for (int o = 0; o < a.prog.n_outputs; ++o) store_unit<TO, E>(a.out[o], unit * E, reg[a.prog.out_reg[o]]);
  }
}

// Scalar interpreter: any dtype mix, any alignment, any broadcast mode; also the tail
// of the vector paths.  Elements [a.first, a.n).
__global__ void __launch_bounds__(kThreads) ew_interp_scalar_f_kernel(const __grid_constant__ EwArgs a) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  float reg[kMaxRegs][1];
  for (int64_t i = a.first + static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < a.n; i += stride) {
    for (int k = 0; k < a.prog.n_inputs; ++k)
      reg[k][0] = load_scalar_f(a.in[k], a.in_dtype[k], input_index(a.prog.input_mode[k], i, a.cols));
    interpret_f<1>(a.prog, reg);
    for (int o = 0; o < a.prog.n_outputs; ++o)
      store_scalar_f(a.out[o], a.out_dtype[o], i, reg[a.prog.out_reg[o]][0]);
  }
}

__global__ void __launch_bounds__(kThreads) ew_interp_scalar_i_kernel(const __grid_constant__ EwArgs a) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  int64_t reg[kMaxRegs];
  for (int64_t i = a.first + static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < a.n; i += stride) {
    for (int k = 0; k < a.prog.n_inputs; ++k)
      reg[k] = load_scalar_i(a.in[k], a.in_dtype[k], input_index(a.prog.input_mode[k], i, a.cols));
    for (int k = 0; k < a.prog.n_instr; ++k) {
      const cdr_ew_instr ins = a.prog.instr[k];
      int64_t v = apply_op_i(ins.op, reg[ins.a], reg[ins.b], reg[ins.c], ins.imm);
      if (ins.round_to == CDR_I32) v = static_cast<int32_t>(v);
      reg[a.prog.n_inputs + k] = v;
    }
    for (int o = 0; o < a.prog.n_outputs; ++o) store_scalar_i(a.out[o], a.out_dtype[o], i, reg[a.prog.out_reg[o]]);
  }
}

// ---------------------------------------------------------------- host side
enum NamedChain { kNone = 0, kMulAdd, kMulAddRelu, kAddCDiv1, kRelu, kAdd, kSub, kMul, kDiv };

bool instr_is(const cdr_ew_instr& i, int op, int a, int b) {
  return i.op == op && i.a == a && i.b == b;
}
bool instr_is_comm(const cdr_ew_instr& i, int op, int a, int b) {
  return i.op == op && ((i.a == a && i.b == b) || (i.a == b && i.b == a));
}

// Recognise the compile-time chains.  `dt` is the dtype every op must round to.
NamedChain match_named(const cdr_ew_params& p, int dt) {
  if (p.n_outputs != 1) return kNone;
  for (int k = 0; k < p.n_instr; ++k)
    if (p.instr[k].round_to != dt) return kNone;
  const int n = p.n_inputs;
  if (p.out_reg[0] != n + p.n_instr - 1) return kNone;
  if (n == 3 && p.n_instr == 2 && instr_is_comm(p.instr[0], CDR_OP_MUL, 0, 1) &&
      instr_is_comm(p.instr[1], CDR_OP_ADD, 3, 2))
    return kMulAdd;
  if (n == 3 && p.n_instr == 3 && instr_is_comm(p.instr[0], CDR_OP_MUL, 0, 1) &&
      instr_is_comm(p.instr[1], CDR_OP_ADD, 3, 2) && p.instr[2].op == CDR_OP_RELU && p.instr[2].a == 4)
    return kMulAddRelu;
  if (n == 3 && p.n_instr == 1 && p.instr[0].op == CDR_OP_ADDCDIV && p.instr[0].a == 0 &&
      p.instr[0].b == 1 && p.instr[0].c == 2 && p.instr[0].imm == 1.0f)
    return kAddCDiv1;
  if (n == 1 && p.n_instr == 1 && p.instr[0].op == CDR_OP_RELU && p.instr[0].a == 0) return kRelu;
  if (n == 2 && p.n_instr == 1) {
    if (instr_is_comm(p.instr[0], CDR_OP_ADD, 0, 1)) return kAdd;
    if (instr_is(p.instr[0], CDR_OP_SUB, 0, 1)) return kSub;
    if (instr_is_comm(p.instr[0], CDR_OP_MUL, 0, 1)) return kMul;
    if (instr_is(p.instr[0], CDR_OP_DIV, 0, 1)) return kDiv;
  }
  return kNone;
}

template <class Chain, typename T>
int launch_named(const EwArgs& a, int64_t n_units, cudaStream_t s) {
  constexpr int UNROLL = (sizeof(T) == 4) ? 4 : 1;
  const int64_t per_cta = static_cast<int64_t>(kThreads) * UNROLL;
  const int64_t grid = (n_units + per_cta - 1) / per_cta;
  if (grid > 0x7fffffff) { set_error("elementwise: tensor too large for one launch"); return CDR_ERR_UNSUPPORTED; }
  bool all_full = true;
  for (int i = 0; i < Chain::NIN; ++i) all_full &= a.prog.input_mode[i] == CDR_IN_FULL;
  if (all_full) ew_named_kernel<Chain, T, T, UNROLL, true><<<static_cast<unsigned>(grid), kThreads, 0, s>>>(a);
  else ew_named_kernel<Chain, T, T, UNROLL, false><<<static_cast<unsigned>(grid), kThreads, 0, s>>>(a);
  return CDR_OK;
}

template <typename T>
int dispatch_named(NamedChain c, const EwArgs& a, int64_t n_units, cudaStream_t s) {
  switch (c) {
    case kMulAdd: return launch_named<ChainMulAdd<T>, T>(a, n_units, s);
    case kMulAddRelu: return launch_named<ChainMulAddRelu<T>, T>(a, n_units, s);
    case kAddCDiv1: return launch_named<ChainAddCDiv1<T>, T>(a, n_units, s);
    case kRelu: return launch_named<ChainRelu<T>, T>(a, n_units, s);
    case kAdd: return launch_named<ChainBinary<T, CDR_OP_ADD>, T>(a, n_units, s);
    case kSub: return launch_named<ChainBinary<T, CDR_OP_SUB>, T>(a, n_units, s);
    case kMul: return launch_named<ChainBinary<T, CDR_OP_MUL>, T>(a, n_units, s);
    case kDiv: return launch_named<ChainBinary<T, CDR_OP_DIV>, T>(a, n_units, s);
    default: return CDR_ERR_UNSUPPORTED;
  }
}

template <typename T, typename TO>
void launch_interp_vec(const EwArgs& a, int64_t n_units, cudaStream_t s) {
  int64_t grid = (n_units + kThreads - 1) / kThreads;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  if (grid > cap) grid = cap;
  ew_interp_vec_kernel<T, TO><<<static_cast<unsigned>(grid), kThreads, 0, s>>>(a);
}

bool is_float_dtype(int dt) { return dt == CDR_F32 || dt == CDR_BF16 || dt == CDR_F16; }
bool is_int_dtype(int dt) { return dt == CDR_I32 || dt == CDR_I64 || dt == CDR_BOOL; }

}  // namespace

int validate_ew_program(const cdr_ew_params* p, int n_in, int n_out) {
  if (!p) { set_error("elementwise: params is null"); return CDR_ERR_BAD_ARG; }
  if (p->n_inputs != n_in || n_in < 0 || n_in > CDR_EW_MAX_INPUTS) {
    set_error("elementwise: program expects %d inputs, call passes %d", p->n_inputs, n_in);
    return CDR_ERR_BAD_ARG;
  }
  if (p->n_outputs != n_out || n_out < 1 || n_out > CDR_EW_MAX_OUTPUTS) {
    set_error("elementwise: program declares %d outputs, call passes %d", p->n_outputs, n_out);
    return CDR_ERR_BAD_ARG;
  }
  if (p->n_instr < 0 || p->n_instr > CDR_EW_MAX_INSTR) {
    set_error("elementwise: %d instructions (max %d)", p->n_instr, CDR_EW_MAX_INSTR);
    return CDR_ERR_BAD_ARG;
  }
  for (int k = 0; k < p->n_instr; ++k) {
    const cdr_ew_instr& i = p->instr[k];
    const int limit = n_in + k;  // only earlier registers may be read
    if (i.op < CDR_OP_ADD || i.op > CDR_OP_LAST) {
      set_error("elementwise: instruction %d has unknown op %d", k, i.op);
      return CDR_ERR_UNSUPPORTED;
    }
    if (i.a < 0 || i.b < 0 || i.c < 0 || (limit > 0 && (i.a >= limit || i.b >= limit || i.c >= limit)) ||
        (limit == 0 && (i.a | i.b | i.c) != 0)) {
      set_error("elementwise: instruction %d reads a register that is not defined yet", k);
      return CDR_ERR_BAD_ARG;
    }
  }
  for (int o = 0; o < n_out; ++o)
    if (p->out_reg[o] < 0 || p->out_reg[o] >= n_in + p->n_instr) {
      set_error("elementwise: output %d names register %d (have %d)", o, p->out_reg[o], n_in + p->n_instr);
      return CDR_ERR_BAD_ARG;
    }
  for (int i = 0; i < n_in; ++i)
    if (p->input_mode[i] < CDR_IN_FULL || p->input_mode[i] > CDR_IN_SCALAR) {
      set_error("elementwise: input %d has unknown broadcast mode %d", i, p->input_mode[i]);
      return CDR_ERR_BAD_ARG;
    }
  return CDR_OK;
}

// Expected element count of an input under its broadcast mode.
int64_t expected_input_numel(int mode, int64_t n, int64_t cols) {
  switch (mode) {
    case CDR_IN_FULL: return n;
    case CDR_IN_ROW: return cols;
    case CDR_IN_COL: return cols ? n / cols : 0;
    default: return 1;
  }
}

int launch_elementwise(const cdr_tensor* ins, int n_in, const cdr_tensor* outs, int n_out,
                       const cdr_ew_params* p, cudaStream_t stream) {
  if (int rc = validate_ew_program(p, n_in, n_out)) return rc;
  const cdr_tensor& out0 = outs[0];
  const int64_t n = numel(out0);
  const int64_t cols = out0.rank > 0 ? out0.shape[out0.rank - 1] : 1;
  for (int o = 0; o < n_out; ++o) {
    if (!outs[o].data && n) { set_error("elementwise: output %d has a null pointer", o); return CDR_ERR_BAD_ARG; }
    if (numel(outs[o]) != n || !is_contiguous(outs[o])) {
      set_error("elementwise: output %d must be contiguous with %lld elements", o, (long long)n);
      return CDR_ERR_BAD_ARG;
    }
  }
  for (int i = 0; i < n_in; ++i) {
    if (!ins[i].data && n) { set_error("elementwise: input %d has a null pointer", i); return CDR_ERR_BAD_ARG; }
    if (!is_contiguous(ins[i])) { set_error("elementwise: input %d is not contiguous", i); return CDR_ERR_BAD_ARG; }
    if (numel(ins[i]) != expected_input_numel(p->input_mode[i], n, cols)) {
      set_error("elementwise: input %d has %lld elements, broadcast mode %d needs %lld", i,
                (long long)numel(ins[i]), p->input_mode[i],
                (long long)expected_input_numel(p->input_mode[i], n, cols));
      return CDR_ERR_BAD_ARG;
    }
  }
  if (n == 0) return CDR_OK;

  EwArgs a{};
  for (int i = 0; i < n_in; ++i) { a.in[i] = ins[i].data; a.in_dtype[i] = ins[i].dtype; }
  for (int o = 0; o < n_out; ++o) { a.out[o] = outs[o].data; a.out_dtype[o] = outs[o].dtype; }
  a.n = n; a.cols = cols; a.first = 0; a.prog = *p;

  bool all_float = true, all_int = true;
  for (int i = 0; i < n_in; ++i) { all_float &= is_float_dtype(ins[i].dtype); all_int &= is_int_dtype(ins[i].dtype); }
  for (int o = 0; o < n_out; ++o) { all_float &= is_float_dtype(outs[o].dtype); all_int &= is_int_dtype(outs[o].dtype); }

  const int64_t scalar_cap = static_cast<int64_t>(sm_count()) * 8;
  if (all_int) {
    for (int k = 0; k < p->n_instr; ++k) {
      const int op = p->instr[k].op;
      const bool ok = op == CDR_OP_ADD || op == CDR_OP_SUB || op == CDR_OP_MUL || op == CDR_OP_RELU ||
                      op == CDR_OP_NEG || op == CDR_OP_ABS || op == CDR_OP_MAX || op == CDR_OP_MIN ||
                      op == CDR_OP_ADDCMUL || op == CDR_OP_CONST || op == CDR_OP_COPY ||
                      op == CDR_OP_ADD_IMM || op == CDR_OP_MUL_IMM || op == CDR_OP_RSUB_IMM ||
                      (op >= CDR_OP_GT && op <= CDR_OP_WHERE);
      if (!ok) { set_error("elementwise: op %d has no integer form", op); return CDR_ERR_UNSUPPORTED; }
    }
    int64_t grid = (n + kThreads - 1) / kThreads;
    if (grid > scalar_cap) grid = scalar_cap;
    ew_interp_scalar_i_kernel<<<static_cast<unsigned>(grid), kThreads, 0, stream>>>(a);
    CDR_CUDA_TRY(cudaGetLastError());
    return CDR_OK;
  }
  if (!all_float) {
    // Mixed clusters (a bool mask selecting between float tensors, a comparison whose result leaves
    // the cluster as bool, an integer tensor scaling a float one).  With only float and bool
    // operands the run-time instance handles them (flags travel as bytes, registers are fp32);
    // anything else, and the tail, goes through the scalar interpreter, which converts every
    // input to fp32 registers and every output from them.
    int64_t done = 0;
    bool flags_only = true, any16 = false;
    for (int i = 0; i < n_in; ++i) { flags_only &= is_float_dtype(ins[i].dtype) || ins[i].dtype == CDR_BOOL; any16 |= dtype_size(ins[i].dtype) == 2; }
    for (int o = 0; o < n_out; ++o) { flags_only &= is_float_dtype(outs[o].dtype) || outs[o].dtype == CDR_BOOL; any16 |= dtype_size(outs[o].dtype) == 2; }
    const int EJ = any16 ? 8 : 4;
    bool jit_ok = flags_only && n >= EJ;
    for (int o = 0; o < n_out; ++o) jit_ok &= aligned16(outs[o].data);
    for (int i = 0; i < n_in; ++i) {
      const int m = p->input_mode[i];
      if (m == CDR_IN_FULL || m == CDR_IN_ROW) jit_ok &= aligned16(ins[i].data);
      if (m == CDR_IN_ROW || m == CDR_IN_COL) jit_ok &= (cols % EJ == 0);
    }
    if (jit_ok) {
      const int rc = launch_elementwise_jit(a.in, a.out, a.in_dtype, a.out_dtype, *p, n / EJ, cols, EJ, stream);
      if (rc == CDR_OK) done = (n / EJ) * EJ;
      else if (rc != CDR_ERR_UNSUPPORTED) return rc;
    }
    if (done < n) {
      a.first = done;
      int64_t grid = (n - done + kThreads - 1) / kThreads;
      if (grid > scalar_cap) grid = scalar_cap;
      ew_interp_scalar_f_kernel<<<static_cast<unsigned>(grid), kThreads, 0, stream>>>(a);
      CDR_CUDA_TRY(cudaGetLastError());
    }
    return CDR_OK;
  }

  // Vector path needs: one dtype for all inputs, one for all outputs, 16-byte aligned
  // pointers, and row-broadcast inputs whose row length is a multiple of the unit.
  bool uniform = true;
  const int in_dt = n_in ? ins[0].dtype : outs[0].dtype;
  for (int i = 0; i < n_in; ++i) uniform &= ins[i].dtype == in_dt;
  for (int o = 0; o < n_out; ++o) uniform &= outs[o].dtype == outs[0].dtype;
  const int out_dt = outs[0].dtype;
  const int vi = 16 / dtype_size(in_dt), vo = 16 / dtype_size(out_dt);
  const int E = vi > vo ? vi : vo;
  bool vec_ok = uniform;
  for (int o = 0; o < n_out; ++o) vec_ok &= aligned16(outs[o].data);
  for (int i = 0; i < n_in; ++i) {
    const int m = p->input_mode[i];
    if (m == CDR_IN_FULL || m == CDR_IN_ROW) vec_ok &= aligned16(ins[i].data);
    if (m == CDR_IN_ROW || m == CDR_IN_COL) vec_ok &= (cols % E == 0);
  }

  int64_t done = 0;
  // A program without an ahead-of-time instance is instantiated at run time (NVRTC); inputs may
  // then have different float dtypes.  CDR_ERR_UNSUPPORTED from the JIT means "not available".
  {
    bool any16 = false, jit_ok = true;
    for (int i = 0; i < n_in; ++i) any16 |= dtype_size(ins[i].dtype) == 2;
    for (int o = 0; o < n_out; ++o) any16 |= dtype_size(outs[o].dtype) == 2;
    const int EJ = any16 ? 8 : 4;
    for (int o = 0; o < n_out; ++o) jit_ok &= aligned16(outs[o].data);
    for (int i = 0; i < n_in; ++i) {
      const int m = p->input_mode[i];
      if (m == CDR_IN_FULL || m == CDR_IN_ROW) jit_ok &= aligned16(ins[i].data);
      if (m == CDR_IN_ROW || m == CDR_IN_COL) jit_ok &= (cols % EJ == 0);
    }
    const bool named = vec_ok && in_dt == out_dt && match_named(*p, in_dt) != kNone;
    if (jit_ok && !named && n >= EJ) {
      const int rc = launch_elementwise_jit(a.in, a.out, a.in_dtype, a.out_dtype, *p, n / EJ, cols, EJ, stream);
      if (rc == CDR_OK) done = (n / EJ) * EJ;
      else if (rc != CDR_ERR_UNSUPPORTED) return rc;
    }
  }
  if (done == 0 && vec_ok && n >= E) {
    const int64_t n_units = n / E;
    const NamedChain c = (in_dt == out_dt) ? match_named(*p, in_dt) : kNone;
    int rc = CDR_ERR_UNSUPPORTED;
    if (c != kNone) {
      if (in_dt == CDR_F32) rc = dispatch_named<float>(c, a, n_units, stream);
      else if (in_dt == CDR_BF16) rc = dispatch_named<__nv_bfloat16>(c, a, n_units, stream);
      else rc = dispatch_named<__half>(c, a, n_units, stream);
      if (rc != CDR_OK && rc != CDR_ERR_UNSUPPORTED) return rc;
    }
    if (rc != CDR_OK) {
      rc = CDR_OK;
#define CDR_EW_VEC(TI, TO) launch_interp_vec<TI, TO>(a, n_units, stream)
      if (in_dt == CDR_F32 && out_dt == CDR_F32) CDR_EW_VEC(float, float);
      else if (in_dt == CDR_BF16 && out_dt == CDR_BF16) CDR_EW_VEC(__nv_bfloat16, __nv_bfloat16);
      else if (in_dt == CDR_F16 && out_dt == CDR_F16) CDR_EW_VEC(__half, __half);
      else if (in_dt == CDR_BF16 && out_dt == CDR_F32) CDR_EW_VEC(__nv_bfloat16, float);
      else if (in_dt == CDR_F16 && out_dt == CDR_F32) CDR_EW_VEC(__half, float);
      else if (in_dt == CDR_F32 && out_dt == CDR_BF16) CDR_EW_VEC(float, __nv_bfloat16);
      else if (in_dt == CDR_F32 && out_dt == CDR_F16) CDR_EW_VEC(float, __half);
      else rc = CDR_ERR_UNSUPPORTED;
#undef CDR_EW_VEC
    }
    if (rc == CDR_OK) {
      CDR_CUDA_TRY(cudaGetLastError());
      done = n_units * E;
    }
  }
  if (done < n) {
    a.first = done;
    int64_t grid = (n - done + kThreads - 1) / kThreads;
    if (grid > scalar_cap) grid = scalar_cap;
    ew_interp_scalar_f_kernel<<<static_cast<unsigned>(grid), kThreads, 0, stream>>>(a);
    CDR_CUDA_TRY(cudaGetLastError());
  }
  return CDR_OK;
}

}  // namespace cdr
