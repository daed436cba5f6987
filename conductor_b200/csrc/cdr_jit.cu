// Runtime instantiation of the elementwise-chain template for programs that have no
// ahead-of-time instance.
//
// The reference prints a whole Choreo program per graph and shells out to a compiler
// (conductor/compiler/jit_compiler.py:235-382).  Here only the chain body is generated: a fixed,
// hand-written kernel skeleton (128-bit streaming loads of every input up front, values in
// registers, 128-bit streaming stores) is specialised with the cluster's straight-line program,
// compiled for sm_100a with NVRTC (no headers, ~0.1 s), loaded through the driver API and cached
// per device.  Arithmetic is the same as everywhere else: fp32 ops rounded one by one, no fma
// contraction, each result rounded to the op's dtype.  If NVRTC or the driver entry points are
// not available the caller falls back to the register-file interpreter kernel.
#include <cuda.h>
#include <dlfcn.h>
#include <nvrtc.h>
#include <stdio.h>
#include <stdlib.h>

#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "cdr_common.cuh"

namespace cdr {
namespace {

// ---------------------------------------------------------------- NVRTC / driver bindings
struct Api {
  bool ok = false;
  nvrtcResult (*CreateProgram)(nvrtcProgram*, const char*, const char*, int, const char* const*, const char* const*);
  nvrtcResult (*CompileProgram)(nvrtcProgram, int, const char* const*);
  nvrtcResult (*GetCUBINSize)(nvrtcProgram, size_t*);
  nvrtcResult (*GetCUBIN)(nvrtcProgram, char*);
  nvrtcResult (*GetProgramLogSize)(nvrtcProgram, size_t*);
  nvrtcResult (*GetProgramLog)(nvrtcProgram, char*);
  nvrtcResult (*DestroyProgram)(nvrtcProgram*);
  CUresult (*ModuleLoadData)(CUmodule*, const void*);
  CUresult (*ModuleGetFunction)(CUfunction*, CUmodule, const char*);
  CUresult (*LaunchKernel)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, CUstream,
                           void**, void**);
};

void* driver_entry(const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
    return nullptr;
  return p;
}

const Api& api() {
  static Api a;
  static std::once_flag once;
  std::call_once(once, [] {
    if (getenv("CDR_DISABLE_JIT")) return;
    void* h = dlopen("libnvrtc.so.12", RTLD_NOW | RTLD_LOCAL);
    if (!h) h = dlopen("libnvrtc.so", RTLD_NOW | RTLD_LOCAL);
    if (!h) return;
#define CDR_SYM(field, name) \
  a.field = reinterpret_cast<decltype(a.field)>(dlsym(h, name)); \
  if (!a.field) return;
    CDR_SYM(CreateProgram, "nvrtcCreateProgram")
    CDR_SYM(CompileProgram, "nvrtcCompileProgram")
    CDR_SYM(GetCUBINSize, "nvrtcGetCUBINSize")
    CDR_SYM(GetCUBIN, "nvrtcGetCUBIN")
    CDR_SYM(GetProgramLogSize, "nvrtcGetProgramLogSize")
    CDR_SYM(GetProgramLog, "nvrtcGetProgramLog")
    CDR_SYM(DestroyProgram, "nvrtcDestroyProgram")
#undef CDR_SYM
    a.ModuleLoadData = reinterpret_cast<decltype(a.ModuleLoadData)>(driver_entry("cuModuleLoadData"));
    a.ModuleGetFunction = reinterpret_cast<decltype(a.ModuleGetFunction)>(driver_entry("cuModuleGetFunction"));
    a.LaunchKernel = reinterpret_cast<decltype(a.LaunchKernel)>(driver_entry("cuLaunchKernel"));
    a.ok = a.ModuleLoadData && a.ModuleGetFunction && a.LaunchKernel;
  });
  return a;
}

// ---------------------------------------------------------------- source generation
const char* kPrelude = R"SRC(
typedef unsigned int u32; typedef unsigned short u16; typedef long long i64;
struct __align__(16) U4 { u32 x, y, z, w; };
struct Args { const void* in[8]; void* out[4]; i64 n_units; i64 cols; };
__device__ __forceinline__ U4 ld_cs(const void* p) { U4 v; asm volatile("ld.global.cs.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p)); return v; }
__device__ __forceinline__ U4 ld_nc(const void* p) { U4 v; asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p)); return v; }
__device__ __forceinline__ void st_cs(void* p, U4 v) { asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" :: "l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory"); }
__device__ __forceinline__ float bf2f(u32 h) { return __uint_as_float(h << 16); }
__device__ __forceinline__ u32 f2bf(float x) { u16 h; asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(h) : "f"(x)); return h; }
__device__ __forceinline__ float h2f(u32 h) { float f; u16 s = (u16)h; asm("cvt.f32.f16 %0, %1;" : "=f"(f) : "h"(s)); return f; }
__device__ __forceinline__ u32 f2h(float x) { u16 h; asm("cvt.rn.f16.f32 %0, %1;" : "=h"(h) : "f"(x)); return h; }
__device__ __forceinline__ float rnd1(float x) { return bf2f(f2bf(x)); }   // round to bf16
__device__ __forceinline__ float rnd2(float x) { return h2f(f2h(x)); }     // round to f16
__device__ __forceinline__ float rnd0(float x) { return x; }
__device__ __forceinline__ float relu_f(float x) { return x > 0.0f ? x : (x != x ? x : 0.0f); }
__device__ __forceinline__ float max_f(float a, float b) { return (a != a || b != b) ? (a + b) : fmaxf(a, b); }
__device__ __forceinline__ float min_f(float a, float b) { return (a != a || b != b) ? (a + b) : fminf(a, b); }
__device__ __forceinline__ void un_f32(U4 q, float* f) { f[0] = __uint_as_float(q.x); f[1] = __uint_as_float(q.y); f[2] = __uint_as_float(q.z); f[3] = __uint_as_float(q.w); }
__device__ __forceinline__ void un_bf16(U4 q, float* f) { u32 w[4] = {q.x, q.y, q.z, q.w}; for (int i = 0; i < 4; ++i) { f[2*i] = __uint_as_float(w[i] << 16); f[2*i+1] = __uint_as_float(w[i] & 0xffff0000u); } }
__device__ __forceinline__ void un_f16(U4 q, float* f) { u32 w[4] = {q.x, q.y, q.z, q.w}; for (int i = 0; i < 4; ++i) { f[2*i] = h2f(w[i] & 0xffffu); f[2*i+1] = h2f(w[i] >> 16); } }
__device__ __forceinline__ U4 pk_f32(const float* f) { U4 q; q.x = __float_as_uint(f[0]); q.y = __float_as_uint(f[1]); q.z = __float_as_uint(f[2]); q.w = __float_as_uint(f[3]); return q; }
__device__ __forceinline__ U4 pk_bf16(const float* f) { u32 w[4]; for (int i = 0; i < 4; ++i) w[i] = f2bf(f[2*i]) | (f2bf(f[2*i+1]) << 16); U4 q; q.x = w[0]; q.y = w[1]; q.z = w[2]; q.w = w[3]; return q; }
__device__ __forceinline__ u32 ld_cs32(const void* p) { u32 v; asm volatile("ld.global.cs.u32 %0, [%1];" : "=r"(v) : "l"(p)); return v; }
__device__ __forceinline__ void st_cs32(void* p, u32 v) { asm volatile("st.global.cs.u32 [%0], %1;" :: "l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ void un_bool4(u32 w, float* f) { for (int i = 0; i < 4; ++i) f[i] = ((w >> (8 * i)) & 0xffu) ? 1.0f : 0.0f; }
__device__ __forceinline__ u32 pk_bool4(const float* f) { u32 w = 0; for (int i = 0; i < 4; ++i) w |= (f[i] != 0.0f ? 1u : 0u) << (8 * i); return w; }
__device__ __forceinline__ u32 badd(u32 a, u32 b) { u32 d; asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }
__device__ __forceinline__ u32 bsub(u32 a, u32 b) { u32 d; asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }
__device__ __forceinline__ u32 bmul(u32 a, u32 b) { u32 d; asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }
__device__ __forceinline__ u32 bmax(u32 a, u32 b) { u32 d; asm("max.NaN.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }
__device__ __forceinline__ u32 bmin(u32 a, u32 b) { u32 d; asm("min.NaN.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }
__device__ __forceinline__ u32 bneg(u32 a) { u32 d; asm("neg.bf16x2 %0, %1;" : "=r"(d) : "r"(a)); return d; }
__device__ __forceinline__ u32 babs(u32 a) { u32 d; asm("abs.bf16x2 %0, %1;" : "=r"(d) : "r"(a)); return d; }
__device__ __forceinline__ U4 pk_f16(const float* f) { u32 w[4]; for (int i = 0; i < 4; ++i) w[i] = f2h(f[2*i]) | (f2h(f[2*i+1]) << 16); U4 q; q.x = w[0]; q.y = w[1]; q.z = w[2]; q.w = w[3]; return q; }
)SRC";

const char* dt_c(int dt) { return dt == CDR_F32 ? "float" : dt == CDR_BOOL ? "unsigned char" : "u16"; }
const char* dt_un(int dt) { return dt == CDR_F32 ? "un_f32" : dt == CDR_BF16 ? "un_bf16" : "un_f16"; }
const char* dt_pk(int dt) { return dt == CDR_F32 ? "pk_f32" : dt == CDR_BF16 ? "pk_bf16" : "pk_f16"; }
const char* dt_scalar(int dt) { return dt == CDR_F32 ? "" : dt == CDR_BF16 ? "bf2f" : dt == CDR_BOOL ? "(float)" : "h2f"; }
int dt_vec(int dt) { return dt == CDR_F32 ? 4 : 8; }

std::string fimm(float v) {
  char buf[64];
  unsigned bits;
  memcpy(&bits, &v, 4);
  snprintf(buf, sizeof(buf), "__uint_as_float(0x%08xu)", bits);   // exact, also for inf / nan
  return buf;
}

std::string expr(const cdr_ew_instr& i) {
  auto R = [](int r) { return "r" + std::to_string(r); };
  const std::string a = R(i.a), b = R(i.b), c = R(i.c), k = fimm(i.imm);
  switch (i.op) {
    case CDR_OP_ADD: return "__fadd_rn(" + a + ", " + b + ")";
    case CDR_OP_SUB: return "__fsub_rn(" + a + ", " + b + ")";
    case CDR_OP_MUL: return "__fmul_rn(" + a + ", " + b + ")";
    case CDR_OP_DIV: return "__fdiv_rn(" + a + ", " + b + ")";
    case CDR_OP_RELU: return "relu_f(" + a + ")";
    case CDR_OP_NEG: return "(-" + a + ")";
    case CDR_OP_ABS: return "fabsf(" + a + ")";
    case CDR_OP_EXP: return "expf(" + a + ")";
    case CDR_OP_LOG: return "logf(" + a + ")";
    case CDR_OP_SQRT: return "__fsqrt_rn(" + a + ")";
    case CDR_OP_SIGMOID: return "__fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-" + a + ")))";
    case CDR_OP_TANH: return "tanhf(" + a + ")";
    case CDR_OP_SIN: return "sinf(" + a + ")";
    case CDR_OP_COS: return "cosf(" + a + ")";
    case CDR_OP_MAX: return "max_f(" + a + ", " + b + ")";
    case CDR_OP_MIN: return "min_f(" + a + ", " + b + ")";
    case CDR_OP_ADDCDIV: return "__fadd_rn(" + a + ", __fdiv_rn(__fmul_rn(" + k + ", " + b + "), " + c + "))";
    case CDR_OP_ADDCMUL: return "__fadd_rn(" + a + ", __fmul_rn(__fmul_rn(" + k + ", " + b + "), " + c + "))";
    case CDR_OP_CONST: return k;
    case CDR_OP_COPY: return a;
    case CDR_OP_ADD_IMM: return "__fadd_rn(" + a + ", " + k + ")";
    case CDR_OP_MUL_IMM: return "__fmul_rn(" + a + ", " + k + ")";
    case CDR_OP_RSUB_IMM: return "__fsub_rn(" + k + ", " + a + ")";
    case CDR_OP_RDIV_IMM: return "__fdiv_rn(" + k + ", " + a + ")";
    case CDR_OP_GT: return "(" + a + " > " + b + " ? 1.0f : 0.0f)";
    case CDR_OP_GE: return "(" + a + " >= " + b + " ? 1.0f : 0.0f)";
    case CDR_OP_LT: return "(" + a + " < " + b + " ? 1.0f : 0.0f)";
    case CDR_OP_LE: return "(" + a + " <= " + b + " ? 1.0f : 0.0f)";
    case CDR_OP_EQ: return "(" + a + " == " + b + " ? 1.0f : 0.0f)";
    case CDR_OP_NE: return "(" + a + " != " + b + " ? 1.0f : 0.0f)";
    case CDR_OP_WHERE: return "(" + a + " != 0.0f ? " + b + " : " + c + ")";
    case CDR_OP_RSQRT: return "__fdiv_rn(1.0f, __fsqrt_rn(" + a + "))";
    case CDR_OP_SILU: return "__fdiv_rn(" + a + ", __fadd_rn(1.0f, expf(-" + a + ")))";
    case CDR_OP_GELU: return "__fmul_rn(__fmul_rn(" + a + ", 0.5f), __fadd_rn(1.0f, erff(__fmul_rn(" + a + ", 0.70710678118654752440f))))";
    case CDR_OP_ERF: return "erff(" + a + ")";
    default: return "0.0f";
  }
}

// The program on one element: registers become local constants, every op rounds to its result type.
std::string chain_source(const cdr_ew_params& p) {
  const int nin = p.n_inputs;
  std::string s = "__device__ __forceinline__ void chain(const float* in, float* out) {\n";
  for (int i = 0; i < nin; ++i) s += "  const float r" + std::to_string(i) + " = in[" + std::to_string(i) + "];\n";
  for (int k = 0; k < p.n_instr; ++k) {
    const int rt = p.instr[k].round_to == CDR_BF16 ? 1 : p.instr[k].round_to == CDR_F16 ? 2 : 0;
    s += "  const float r" + std::to_string(nin + k) + " = rnd" + std::to_string(rt) + "(" + expr(p.instr[k]) + ");\n";
  }
  for (int o = 0; o < p.n_outputs; ++o) s += "  out[" + std::to_string(o) + "] = r" + std::to_string(p.out_reg[o]) + ";\n";
  s += "}\n";
  return s;
}

// Vector loads of input `i` for one unit of E elements into `dst` (FULL and ROW inputs only).
std::string vector_loads(int i, int dt, int mode, int E, const std::string& full_base, const std::string& row_base,
                         const std::string& dst, const std::string& indent) {
  const int V = dt_vec(dt);
  const std::string I = std::to_string(i), T = dt_c(dt);
  const std::string base = mode == CDR_IN_FULL ? full_base : row_base;
  const std::string ld = mode == CDR_IN_FULL ? "ld_cs" : "ld_nc";
  std::string s;
  if (dt == CDR_BOOL) {   // one byte per element: 32-bit loads of four flags
    for (int k = 0; k < E / 4; ++k)
      s += indent + "un_bool4(ld_cs32((const unsigned char*)a.in[" + I + "] + " + base + " + " + std::to_string(k * 4) + "), " + dst +
           " + " + std::to_string(k * 4) + ");\n";
    return s;
  }
  for (int k = 0; k < E / V; ++k)
    s += indent + dt_un(dt) + "(" + ld + "((const " + T + "*)a.in[" + I + "] + " + base + " + " + std::to_string(k * V) + "), " +
         dst + " + " + std::to_string(k * V) + ");\n";
  return s;
}


// ---- packed mode: a chain whose inputs and every op result are bf16 runs on bf16x2 instructions.
// Bit-identical to eager's fp32-then-round: the product of two bf16 values is exact in fp32, and
// an fp32 sum of two bf16 values is either exact or so far from a bf16 tie that rounding once or
// twice gives the same result; max/min/relu propagate NaN (max.NaN); half the instructions of the
// unpack / fp32 op / round sequence.
bool bf16_exact(float v) {
  unsigned bits;
  memcpy(&bits, &v, 4);
  return (bits & 0xffffu) == 0;
}
bool can_pack(const cdr_ew_params& p, const int* in_dt) {
  for (int i = 0; i < p.n_inputs; ++i)
    if (in_dt[i] != CDR_BF16) return false;
  for (int k = 0; k < p.n_instr; ++k) {
    const cdr_ew_instr& in = p.instr[k];
    if (in.round_to != CDR_BF16) return false;
    switch (in.op) {
      case CDR_OP_ADD: case CDR_OP_SUB: case CDR_OP_MUL: case CDR_OP_RELU: case CDR_OP_NEG: case CDR_OP_ABS:
      case CDR_OP_MAX: case CDR_OP_MIN: case CDR_OP_COPY:
        break;
      case CDR_OP_CONST: case CDR_OP_ADD_IMM: case CDR_OP_MUL_IMM: case CDR_OP_RSUB_IMM:
        if (!bf16_exact(in.imm)) return false;
        break;
      default:
        return false;
    }
  }
  return true;
}
std::string pimm(float v) {
  unsigned bits;
  memcpy(&bits, &v, 4);
  char buf[32];
  snprintf(buf, sizeof(buf), "0x%08xu", (bits >> 16) | (bits & 0xffff0000u));
  return buf;
}
std::string pexpr(const cdr_ew_instr& i) {
  auto R = [](int r) { return "r" + std::to_string(r); };
  const std::string a = R(i.a), b = R(i.b), k = pimm(i.imm);
  switch (i.op) {
    case CDR_OP_ADD: return "badd(" + a + ", " + b + ")";
    case CDR_OP_SUB: return "bsub(" + a + ", " + b + ")";
    case CDR_OP_MUL: return "bmul(" + a + ", " + b + ")";
    case CDR_OP_RELU: return "bmax(" + a + ", 0u)";
    case CDR_OP_NEG: return "bneg(" + a + ")";
    case CDR_OP_ABS: return "babs(" + a + ")";
    case CDR_OP_MAX: return "bmax(" + a + ", " + b + ")";
    case CDR_OP_MIN: return "bmin(" + a + ", " + b + ")";
    case CDR_OP_CONST: return k;
    case CDR_OP_COPY: return a;
    case CDR_OP_ADD_IMM: return "badd(" + a + ", " + k + ")";
    case CDR_OP_MUL_IMM: return "bmul(" + a + ", " + k + ")";
    case CDR_OP_RSUB_IMM: return "bsub(" + k + ", " + a + ")";
    default: return "0u";
  }
}
// The program on one pair of elements.
std::string chain_source_packed(const cdr_ew_params& p) {
  const int nin = p.n_inputs;
  std::string s = "__device__ __forceinline__ void chain(const u32* in, u32* out) {\n";
  for (int i = 0; i < nin; ++i) s += "  const u32 r" + std::to_string(i) + " = in[" + std::to_string(i) + "];\n";
  for (int k = 0; k < p.n_instr; ++k) s += "  const u32 r" + std::to_string(nin + k) + " = " + pexpr(p.instr[k]) + ";\n";
  for (int o = 0; o < p.n_outputs; ++o) s += "  out[" + std::to_string(o) + "] = r" + std::to_string(p.out_reg[o]) + ";\n";
  s += "}\n";
  return s;
}
// Loads of input `i` for one unit of 8 bf16 into the U4 `dst`.
std::string packed_load(int i, int mode, const std::string& full_idx, const std::string& row_idx, const std::string& col_idx,
                        const std::string& dst, const std::string& indent) {
  const std::string I = std::to_string(i), base = "(const u16*)a.in[" + I + "]";
  if (mode == CDR_IN_FULL) return indent + dst + " = ld_cs(" + base + " + " + full_idx + ");\n";
  if (mode == CDR_IN_ROW) return indent + dst + " = ld_nc(" + base + " + " + row_idx + ");\n";
  const std::string idx = mode == CDR_IN_COL ? col_idx : "0";
  return indent + "{ const u32 t = (" + base + ")[" + idx + "]; const u32 w = t | (t << 16); " + dst + ".x = w; " + dst + ".y = w; " +
         dst + ".z = w; " + dst + ".w = w; }\n";
}

// Packed elementwise kernel: one unit of 8 bf16 per thread.
std::string generate_packed(const cdr_ew_params& p) {
  std::string s = kPrelude;
  const int nin = p.n_inputs;
  s += chain_source_packed(p);
  s += "extern \"C\" __global__ void __launch_bounds__(256) cdr_jit_k(const __grid_constant__ Args a) {\n";
  s += "  const i64 unit = (i64)blockIdx.x * 256 + threadIdx.x;\n  if (unit >= a.n_units) return;\n  const i64 e0 = unit * 8;\n";
  s += "  U4 v[" + std::to_string(nin > 0 ? nin : 1) + "];\n";
  for (int i = 0; i < nin; ++i) s += packed_load(i, p.input_mode[i], "e0", "(e0 % a.cols)", "(e0 / a.cols)", "v[" + std::to_string(i) + "]", "  ");
  s += "  U4 o[" + std::to_string(p.n_outputs) + "];\n";
  const char* comp[4] = {"x", "y", "z", "w"};
  for (int e = 0; e < 4; ++e) {
    s += "  {\n    u32 in[" + std::to_string(nin > 0 ? nin : 1) + "], out[" + std::to_string(p.n_outputs) + "];\n";
    for (int i = 0; i < nin; ++i) s += "    in[" + std::to_string(i) + "] = v[" + std::to_string(i) + "]." + comp[e] + ";\n";
    s += "    chain(in, out);\n";
    for (int o = 0; o < p.n_outputs; ++o) s += "    o[" + std::to_string(o) + "]." + comp[e] + " = out[" + std::to_string(o) + "];\n";
    s += "  }\n";
  }
  for (int o = 0; o < p.n_outputs; ++o) s += "  st_cs((u16*)a.out[" + std::to_string(o) + "] + e0, o[" + std::to_string(o) + "]);\n";
  s += "}\n";
  return s;
}

// One thread handles UN units of E consecutive elements; all loads first, then math and stores.
std::string generate(const cdr_ew_params& p, const int* in_dt, const int* out_dt, int E, int UN) {
  bool out_bf16 = true;
  for (int o = 0; o < p.n_outputs; ++o) out_bf16 &= out_dt[o] == CDR_BF16;
  if (E == 8 && UN == 1 && out_bf16 && p.n_inputs > 0 && can_pack(p, in_dt)) return generate_packed(p);
  std::string s = kPrelude;
  const int nin = p.n_inputs;
  s += chain_source(p);
  const std::string Es = std::to_string(E), UNs = std::to_string(UN);
  s += "extern \"C\" __global__ void __launch_bounds__(256) cdr_jit_k(const __grid_constant__ Args a) {\n";
  s += "  const i64 unit0 = (i64)blockIdx.x * (256 * " + UNs + ") + threadIdx.x;\n";
  s += "  float v[" + UNs + "][" + std::to_string(nin > 0 ? nin : 1) + "][" + Es + "];\n";
  s += "#pragma unroll\n  for (int u = 0; u < " + UNs + "; ++u) {\n    const i64 unit = unit0 + (i64)u * 256;\n    if (unit < a.n_units) {\n      const i64 e0 = unit * " + Es + ";\n";
  for (int i = 0; i < nin; ++i) {
    const int dt = in_dt[i], m = p.input_mode[i];
    const std::string I = std::to_string(i), T = dt_c(dt);
    if (m == CDR_IN_FULL || m == CDR_IN_ROW) {
      s += vector_loads(i, dt, m, E, "e0", "(e0 % a.cols)", "v[u][" + I + "]", "      ");
    } else {
      const std::string idx = m == CDR_IN_COL ? "(e0 / a.cols)" : "0";
      s += "      { const float t = " + std::string(dt_scalar(dt)) + "(((const " + T + "*)a.in[" + I + "])[" + idx +
           "]);\n#pragma unroll\n        for (int e = 0; e < " + Es + "; ++e) v[u][" + I + "][e] = t; }\n";
    }
  }
  s += "    }\n  }\n";
  s += "#pragma unroll\n  for (int u = 0; u < " + UNs + "; ++u) {\n    const i64 unit = unit0 + (i64)u * 256;\n    if (unit < a.n_units) {\n      const i64 e0 = unit * " + Es + ";\n";
  s += "      float o[" + std::to_string(p.n_outputs) + "][" + Es + "];\n";
  s += "#pragma unroll\n      for (int e = 0; e < " + Es + "; ++e) {\n        float in[" + std::to_string(nin > 0 ? nin : 1) + "], out[" +
       std::to_string(p.n_outputs) + "];\n";
  for (int i = 0; i < nin; ++i) s += "        in[" + std::to_string(i) + "] = v[u][" + std::to_string(i) + "][e];\n";
  s += "        chain(in, out);\n";
  for (int o = 0; o < p.n_outputs; ++o) s += "        o[" + std::to_string(o) + "][e] = out[" + std::to_string(o) + "];\n";
  s += "      }\n";
  for (int o = 0; o < p.n_outputs; ++o) {
    const int dt = out_dt[o], V = dt_vec(dt);
    if (dt == CDR_BOOL) {
      for (int k = 0; k < E / 4; ++k)
        s += "      st_cs32((unsigned char*)a.out[" + std::to_string(o) + "] + e0 + " + std::to_string(k * 4) + ", pk_bool4(o[" +
             std::to_string(o) + "] + " + std::to_string(k * 4) + "));\n";
      continue;
    }
    for (int k = 0; k < E / V; ++k)
      s += "      st_cs((" + std::string(dt_c(dt)) + "*)a.out[" + std::to_string(o) + "] + e0 + " + std::to_string(k * V) + ", " +
           dt_pk(dt) + "(o[" + std::to_string(o) + "] + " + std::to_string(k * V) + "));\n";
  }
  s += "    }\n  }\n}\n";
  return s;
}

// Chain + reduction over the last dimension.  G threads (one warp, or the whole 256-thread CTA)
// share a row; a thread walks its row in chunks of U units of E elements, loads first, then math.
// Args: n_units = rows, out[0] = one value per row.
std::string generate_row_reduce_packed(const cdr_ew_params& p, int out_dt, int reduce_op, int U, int G);

std::string generate_row_reduce(const cdr_ew_params& p, const int* in_dt, int out_dt, int reduce_op, int E, int U, int G) {
  if (E == 8 && can_pack(p, in_dt)) return generate_row_reduce_packed(p, out_dt, reduce_op, U, G);
  std::string s = kPrelude;
  const int nin = p.n_inputs;
  s += chain_source(p);
  const char* ident = reduce_op == CDR_RED_MAX ? "__uint_as_float(0xff800000u)" : reduce_op == CDR_RED_MIN ? "__uint_as_float(0x7f800000u)" : "0.0f";
  const char* comb = reduce_op == CDR_RED_MAX ? "max_f" : reduce_op == CDR_RED_MIN ? "min_f" : "__fadd_rn";
  s += std::string("__device__ __forceinline__ float comb(float x, float y) { return ") + comb + "(x, y); }\n";
  const std::string Es = std::to_string(E), Us = std::to_string(U), Gs = std::to_string(G);
  s += "extern \"C\" __global__ void __launch_bounds__(256) cdr_jit_k(const __grid_constant__ Args a) {\n";
  s += "  constexpr int G = " + Gs + ", RPB = 256 / G, U = " + Us + ", E = " + Es + ";\n";
  s += "  const int tg = threadIdx.x % G;\n";
  s += "  const i64 row = (i64)blockIdx.x * RPB + threadIdx.x / G;\n";
  s += "  const bool live = row < a.n_units;\n";
  s += "  const i64 upr = a.cols / E;\n";
  s += std::string("  float acc = ") + ident + ";\n";
  s += "  if (live) {\n";
  for (int i = 0; i < nin; ++i) {
    const int m = p.input_mode[i];
    if (m == CDR_IN_COL || m == CDR_IN_SCALAR)
      s += "    const float s" + std::to_string(i) + " = " + dt_scalar(in_dt[i]) + "(((const " + dt_c(in_dt[i]) + "*)a.in[" +
           std::to_string(i) + "])[" + (m == CDR_IN_COL ? "row" : "0") + "]);\n";
  }
  s += "    for (i64 u0 = tg; u0 < upr; u0 += (i64)G * U) {\n";
  s += "      float v[U][" + std::to_string(nin) + "][E];\n";
  s += "#pragma unroll\n      for (int u = 0; u < U; ++u) {\n        const i64 unit = u0 + (i64)u * G;\n        if (unit < upr) {\n";
  s += "          const i64 c0 = unit * E;\n          const i64 e0 = row * a.cols + c0;\n";
  for (int i = 0; i < nin; ++i) {
    const int m = p.input_mode[i];
    if (m == CDR_IN_FULL || m == CDR_IN_ROW)
      s += vector_loads(i, in_dt[i], m, E, "e0", "c0", "v[u][" + std::to_string(i) + "]", "          ");
  }
  s += "        }\n      }\n";
  s += "#pragma unroll\n      for (int u = 0; u < U; ++u) {\n        if (u0 + (i64)u * G < upr) {\n";
  s += "#pragma unroll\n          for (int e = 0; e < E; ++e) {\n            float in[" + std::to_string(nin) + "], out[1];\n";
  for (int i = 0; i < nin; ++i) {
    const int m = p.input_mode[i];
    const std::string I = std::to_string(i);
    s += "            in[" + I + "] = " + ((m == CDR_IN_FULL || m == CDR_IN_ROW) ? "v[u][" + I + "][e]" : "s" + I) + ";\n";
  }
  s += "            chain(in, out);\n            acc = comb(acc, out[0]);\n          }\n        }\n      }\n    }\n  }\n";
  s += "#pragma unroll\n  for (int o = 16; o > 0; o >>= 1) acc = comb(acc, __shfl_xor_sync(0xffffffffu, acc, o));\n";
  if (G == 256) {
    s += "  __shared__ float part[8];\n";
    s += "  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;\n  __syncthreads();\n";
    s += "  if (threadIdx.x == 0) {\n    acc = part[0];\n#pragma unroll\n    for (int w = 1; w < 8; ++w) acc = comb(acc, part[w]);\n  }\n";
  }
  s += "  if (live && tg == 0) {\n";
  if (reduce_op == CDR_RED_MEAN) s += "    acc = __fdiv_rn(acc, (float)a.cols);\n";
  if (out_dt == CDR_F32) s += "    ((float*)a.out[0])[row] = acc;\n";
  else s += std::string("    ((u16*)a.out[0])[row] = (u16)") + (out_dt == CDR_BF16 ? "f2bf" : "f2h") + "(acc);\n";
  s += "  }\n}\n";
  return s;
}

// Units of E elements a thread keeps in flight.  Measured on B200: 16-bit units unpack to twice the
// registers, and one unit per thread (7.1 TB/s on a 3-input bf16 chain) beats two (6.2) and four (4.2);
// for fp32 two units are best or equal across chains.
int units_per_thread(int E, int) { return E == 4 ? 2 : 1; }


// Packed chain + reduction over the last dimension (see generate_row_reduce for the skeleton):
// the chain runs on bf16x2 pairs, the reduction accumulates their two halves in fp32.
std::string generate_row_reduce_packed(const cdr_ew_params& p, int out_dt, int reduce_op, int U, int G) {
  std::string s = kPrelude;
  const int nin = p.n_inputs;
  s += chain_source_packed(p);
  const char* ident = reduce_op == CDR_RED_MAX ? "__uint_as_float(0xff800000u)" : reduce_op == CDR_RED_MIN ? "__uint_as_float(0x7f800000u)" : "0.0f";
  const char* comb = reduce_op == CDR_RED_MAX ? "max_f" : reduce_op == CDR_RED_MIN ? "min_f" : "__fadd_rn";
  s += std::string("__device__ __forceinline__ float comb(float x, float y) { return ") + comb + "(x, y); }\n";
  s += "extern \"C\" __global__ void __launch_bounds__(256) cdr_jit_k(const __grid_constant__ Args a) {\n";
  s += "  constexpr int G = " + std::to_string(G) + ", RPB = 256 / G, U = " + std::to_string(U) + ", E = 8;\n";
  s += "  const int tg = threadIdx.x % G;\n";
  s += "  const i64 row = (i64)blockIdx.x * RPB + threadIdx.x / G;\n";
  s += "  const bool live = row < a.n_units;\n";
  s += "  const i64 upr = a.cols / E;\n";
  s += std::string("  float acc0 = ") + ident + ", acc1 = " + ident + ";\n";
  s += "  if (live) {\n";
  s += "    for (i64 u0 = tg; u0 < upr; u0 += (i64)G * U) {\n";
  s += "      U4 v[U][" + std::to_string(nin) + "];\n";
  s += "#pragma unroll\n      for (int u = 0; u < U; ++u) {\n        const i64 unit = u0 + (i64)u * G;\n        if (unit < upr) {\n";
  s += "          const i64 c0 = unit * E;\n          const i64 e0 = row * a.cols + c0;\n";
  for (int i = 0; i < nin; ++i) s += packed_load(i, p.input_mode[i], "e0", "c0", "row", "v[u][" + std::to_string(i) + "]", "          ");
  s += "        }\n      }\n";
  s += "#pragma unroll\n      for (int u = 0; u < U; ++u) {\n        if (u0 + (i64)u * G < upr) {\n";
  const char* comp[4] = {"x", "y", "z", "w"};
  for (int e = 0; e < 4; ++e) {
    s += "          {\n            u32 in[" + std::to_string(nin) + "], out[1];\n";
    for (int i = 0; i < nin; ++i) s += "            in[" + std::to_string(i) + "] = v[u][" + std::to_string(i) + "]." + comp[e] + ";\n";
    s += "            chain(in, out);\n";
    s += "            acc0 = comb(acc0, __uint_as_float(out[0] << 16));\n            acc1 = comb(acc1, __uint_as_float(out[0] & 0xffff0000u));\n          }\n";
  }
  s += "        }\n      }\n    }\n  }\n";
  s += "  float acc = comb(acc0, acc1);\n";
  s += "#pragma unroll\n  for (int o = 16; o > 0; o >>= 1) acc = comb(acc, __shfl_xor_sync(0xffffffffu, acc, o));\n";
  if (G == 256) {
    s += "  __shared__ float part[8];\n";
    s += "  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;\n  __syncthreads();\n";
    s += "  if (threadIdx.x == 0) {\n    acc = part[0];\n#pragma unroll\n    for (int w = 1; w < 8; ++w) acc = comb(acc, part[w]);\n  }\n";
  }
  s += "  if (live && tg == 0) {\n";
  if (reduce_op == CDR_RED_MEAN) s += "    acc = __fdiv_rn(acc, (float)a.cols);\n";
  if (out_dt == CDR_F32) s += "    ((float*)a.out[0])[row] = acc;\n";
  else s += std::string("    ((u16*)a.out[0])[row] = (u16)") + (out_dt == CDR_BF16 ? "f2bf" : "f2h") + "(acc);\n";
  s += "  }\n}\n";
  return s;
}


// Chain + reduction over every element, one launch: a persistent grid walks units of E elements
// (U per thread in flight), every CTA leaves one partial in scratch, and the CTA that draws the
// last ticket folds the partials and writes the result.  Args: n_units = elements / E, out[0] =
// result, out[1] = float partials (one per CTA), out[2] = ticket counter (zero at launch, left zero).
std::string generate_full_reduce(const cdr_ew_params& p, const int* in_dt, int out_dt, int reduce_op, int E, int U) {
  const bool packed = E == 8 && can_pack(p, in_dt);
  std::string s = kPrelude;
  const int nin = p.n_inputs;
  s += packed ? chain_source_packed(p) : chain_source(p);
  const char* ident = reduce_op == CDR_RED_MAX ? "__uint_as_float(0xff800000u)" : reduce_op == CDR_RED_MIN ? "__uint_as_float(0x7f800000u)" : "0.0f";
  const char* comb = reduce_op == CDR_RED_MAX ? "max_f" : reduce_op == CDR_RED_MIN ? "min_f" : "__fadd_rn";
  s += std::string("__device__ __forceinline__ float comb(float x, float y) { return ") + comb + "(x, y); }\n";
  s += "__device__ __forceinline__ float cta_comb(float v, float* part) {\n";
  s += "#pragma unroll\n  for (int o = 16; o > 0; o >>= 1) v = comb(v, __shfl_xor_sync(0xffffffffu, v, o));\n";
  s += "  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = v;\n  __syncthreads();\n";
  s += "  if (threadIdx.x == 0) {\n    v = part[0];\n#pragma unroll\n    for (int w = 1; w < 8; ++w) v = comb(v, part[w]);\n  }\n";
  s += "  __syncthreads();\n  return v;\n}\n";
  s += "extern \"C\" __global__ void __launch_bounds__(256) cdr_jit_k(const __grid_constant__ Args a) {\n";
  s += "  constexpr int U = " + std::to_string(U) + ", E = " + std::to_string(E) + ";\n";
  s += "  __shared__ float part[8];\n  __shared__ int is_last;\n";
  s += "  const i64 stride = (i64)gridDim.x * 256;\n";
  s += std::string("  float acc0 = ") + ident + ", acc1 = " + ident + ";\n";
  s += "  for (i64 base = (i64)blockIdx.x * 256 + threadIdx.x; base < a.n_units; base += stride * U) {\n";
  if (packed) s += "    U4 v[U][" + std::to_string(nin) + "];\n";
  else s += "    float v[U][" + std::to_string(nin) + "][E];\n";
  s += "#pragma unroll\n    for (int u = 0; u < U; ++u) {\n      const i64 unit = base + u * stride;\n      if (unit < a.n_units) {\n        const i64 e0 = unit * E;\n";
  for (int i = 0; i < nin; ++i) {
    const int m = p.input_mode[i];
    const std::string I = std::to_string(i);
    if (packed) {
      s += packed_load(i, m, "e0", "(e0 % a.cols)", "(e0 / a.cols)", "v[u][" + I + "]", "        ");
    } else if (m == CDR_IN_FULL || m == CDR_IN_ROW) {
      s += vector_loads(i, in_dt[i], m, E, "e0", "(e0 % a.cols)", "v[u][" + I + "]", "        ");
    } else {
      const std::string idx = m == CDR_IN_COL ? "(e0 / a.cols)" : "0";
      s += "        { const float t = " + std::string(dt_scalar(in_dt[i])) + "(((const " + dt_c(in_dt[i]) + "*)a.in[" + I + "])[" + idx +
           "]);\n#pragma unroll\n          for (int e = 0; e < E; ++e) v[u][" + I + "][e] = t; }\n";
    }
  }
  s += "      }\n    }\n";
  s += "#pragma unroll\n    for (int u = 0; u < U; ++u) {\n      if (base + u * stride < a.n_units) {\n";
  if (packed) {
    const char* comp[4] = {"x", "y", "z", "w"};
    for (int e = 0; e < 4; ++e) {
      s += "        {\n          u32 in[" + std::to_string(nin) + "], out[1];\n";
      for (int i = 0; i < nin; ++i) s += "          in[" + std::to_string(i) + "] = v[u][" + std::to_string(i) + "]." + comp[e] + ";\n";
      s += "          chain(in, out);\n          acc0 = comb(acc0, __uint_as_float(out[0] << 16));\n          acc1 = comb(acc1, __uint_as_float(out[0] & 0xffff0000u));\n        }\n";
    }
  } else {
    s += "#pragma unroll\n        for (int e = 0; e < E; ++e) {\n          float in[" + std::to_string(nin) + "], out[1];\n";
    for (int i = 0; i < nin; ++i) s += "          in[" + std::to_string(i) + "] = v[u][" + std::to_string(i) + "][e];\n";
    s += "          chain(in, out);\n          if (e & 1) acc1 = comb(acc1, out[0]); else acc0 = comb(acc0, out[0]);\n        }\n";
  }
  s += "      }\n    }\n  }\n";
  s += "  float r = cta_comb(comb(acc0, acc1), part);\n";
  s += "  float* partials = (float*)a.out[1];\n  unsigned int* ticket = (unsigned int*)a.out[2];\n";
  s += "  if (threadIdx.x == 0) {\n    partials[blockIdx.x] = r;\n    __threadfence();\n    is_last = atomicAdd(ticket, 1u) == gridDim.x - 1;\n  }\n";
  s += "  __syncthreads();\n  if (!is_last) return;\n  __threadfence();\n";
  s += std::string("  float acc = ") + ident + ";\n";
  s += "  for (int i = threadIdx.x; i < (int)gridDim.x; i += 256) acc = comb(acc, __ldcg(partials + i));\n";
  s += "  r = cta_comb(acc, part);\n  if (threadIdx.x == 0) {\n";
  if (reduce_op == CDR_RED_MEAN) s += "    r = __fdiv_rn(r, (float)(a.n_units * E));\n";
  if (out_dt == CDR_F32) s += "    ((float*)a.out[0])[0] = r;\n";
  else s += std::string("    ((u16*)a.out[0])[0] = (u16)") + (out_dt == CDR_BF16 ? "f2bf" : "f2h") + "(r);\n";
  s += "    *ticket = 0;\n  }\n}\n";
  return s;
}

struct JitKernel {
  CUfunction fn = nullptr;
  bool failed = false;
};
std::mutex g_mu;
std::unordered_map<std::string, JitKernel> g_cache;   // key: device + source

struct JitArgs {
  const void* in[8];
  void* out[4];
  long long n_units;
  long long cols;
};

}  // namespace

// Source text of the kernel that would be instantiated (for inspection and tests; needs no GPU).
std::string jit_elementwise_source(const cdr_ew_params& p, const int* in_dt, const int* out_dt, int E) {
  return generate(p, in_dt, out_dt, E, units_per_thread(E, p.n_inputs));
}

namespace {
// Row reductions: units a thread keeps in flight, and the threads sharing a row.  A 256-thread CTA
// per row only when every thread then still has a full set of units; otherwise a warp per row, 8
// rows per CTA (C2's shape, 512 units per row, packed chain: 23.8 us with a warp per row against
// 39.3 us with a CTA per row; the hand-tuned ahead-of-time kernel takes 21.1 us).
void reduce_config(const cdr_ew_params& p, const int* in_dt, int E, int64_t cols, int* U, int* G) {
  *U = (E == 8 && can_pack(p, in_dt)) ? 4 : units_per_thread(E, p.n_inputs);
  *G = cols / E >= 256 * *U ? 256 : 32;
}
}  // namespace

std::string jit_full_reduce_source(const cdr_ew_params& p, const int* in_dt, int out_dt, int reduce_op, int E) {
  return generate_full_reduce(p, in_dt, out_dt, reduce_op, E, E == 4 ? 4 : 2);
}

std::string jit_row_reduce_source(const cdr_ew_params& p, const int* in_dt, int out_dt, int reduce_op, int E, int64_t cols) {
  int U, G;
  reduce_config(p, in_dt, E, cols, &U, &G);
  return generate_row_reduce(p, in_dt, out_dt, reduce_op, E, U, G);
}

// Compile `src` to a cubin image for sm_100a; empty on failure (message in `log`).
std::vector<char> jit_compile(const std::string& src, std::string* log) {
  const Api& A = api();
  std::vector<char> cubin;
  if (!A.CreateProgram) { if (log) *log = "NVRTC is not available"; return cubin; }
  nvrtcProgram prog;
  if (A.CreateProgram(&prog, src.c_str(), "cdr_jit.cu", 0, nullptr, nullptr) != NVRTC_SUCCESS) return cubin;
  const char* opts[] = {"--gpu-architecture=sm_100a", "--fmad=false", "--std=c++17"};
  const nvrtcResult rc = A.CompileProgram(prog, 3, opts);
  if (rc != NVRTC_SUCCESS) {
    size_t n = 0;
    if (log && A.GetProgramLogSize(prog, &n) == NVRTC_SUCCESS && n > 1) {
      log->resize(n);
      A.GetProgramLog(prog, &(*log)[0]);
    }
    A.DestroyProgram(&prog);
    return cubin;
  }
  size_t n = 0;
  if (A.GetCUBINSize(prog, &n) == NVRTC_SUCCESS && n > 0) {
    cubin.resize(n);
    if (A.GetCUBIN(prog, cubin.data()) != NVRTC_SUCCESS) cubin.clear();
  }
  A.DestroyProgram(&prog);
  return cubin;
}

namespace {
// Compiled instance of `src` on the current device; CDR_ERR_UNSUPPORTED when there is none.
int get_kernel(const Api& A, const std::string& src, CUfunction* fn) {
  int dev = 0;
  CDR_CUDA_TRY(cudaGetDevice(&dev));
  const std::string key = std::to_string(dev) + "#" + src;
  std::lock_guard<std::mutex> lock(g_mu);
  JitKernel& k = g_cache[key];
  if (k.failed) return CDR_ERR_UNSUPPORTED;
  if (!k.fn) {
    std::string log;
    const std::vector<char> cubin = jit_compile(src, &log);
    CUmodule mod = nullptr;
    if (cubin.empty() || A.ModuleLoadData(&mod, cubin.data()) != CUDA_SUCCESS ||
        A.ModuleGetFunction(&k.fn, mod, "cdr_jit_k") != CUDA_SUCCESS) {
      k.failed = true;
      k.fn = nullptr;
      if (getenv("CDR_JIT_VERBOSE")) fprintf(stderr, "conductor_b200: JIT failed, using the interpreter\n%s\n", log.c_str());
      return CDR_ERR_UNSUPPORTED;
    }
  }
  *fn = k.fn;
  return CDR_OK;
}

int launch_jit(const Api& A, CUfunction fn, JitArgs& args, int64_t grid, cudaStream_t stream, const char* who) {
  if (grid > 0x7fffffff) return CDR_ERR_UNSUPPORTED;
  void* params[] = {&args};
  const CUresult r = A.LaunchKernel(fn, static_cast<unsigned>(grid), 1, 1, 256, 1, 1, 0, reinterpret_cast<CUstream>(stream),
                                    params, nullptr);
  if (r != CUDA_SUCCESS) { set_error("%s: run-time instance launch failed with %d", who, static_cast<int>(r)); return CDR_ERR_CUDA; }
  return CDR_OK;
}
}  // namespace

// Launch the run-time instance for this program on the vector path.  CDR_ERR_UNSUPPORTED means
// "no instance here, use the interpreter"; other non-zero codes are real failures.
int launch_elementwise_jit(const void* const* in, void* const* out, const int* in_dt, const int* out_dt,
                           const cdr_ew_params& p, int64_t n_units, int64_t cols, int E, cudaStream_t stream) {
  const Api& A = api();
  if (!A.ok) return CDR_ERR_UNSUPPORTED;
  const int UN = units_per_thread(E, p.n_inputs);
  CUfunction fn = nullptr;
  if (int rc = get_kernel(A, generate(p, in_dt, out_dt, E, UN), &fn)) return rc;
  JitArgs args{};
  for (int i = 0; i < p.n_inputs; ++i) args.in[i] = in[i];
  for (int o = 0; o < p.n_outputs; ++o) args.out[o] = out[o];
  args.n_units = n_units;
  args.cols = cols;
  const int64_t per_cta = 256LL * UN;
  return launch_jit(A, fn, args, (n_units + per_cta - 1) / per_cta, stream, "elementwise");
}

// Chain + last-dimension reduction; every FULL/ROW input 16-byte aligned and cols % E == 0.
int launch_row_reduce_jit(const void* const* in, void* out, const int* in_dt, int out_dt, const cdr_ew_params& p,
                          int reduce_op, int64_t rows, int64_t cols, int E, cudaStream_t stream) {
  const Api& A = api();
  if (!A.ok) return CDR_ERR_UNSUPPORTED;
  int U, G;
  reduce_config(p, in_dt, E, cols, &U, &G);
  CUfunction fn = nullptr;
  if (int rc = get_kernel(A, generate_row_reduce(p, in_dt, out_dt, reduce_op, E, U, G), &fn)) return rc;
  JitArgs args{};
  for (int i = 0; i < p.n_inputs; ++i) args.in[i] = in[i];
  args.out[0] = out;
  args.n_units = rows;
  args.cols = cols;
  const int64_t rpb = 256 / G;
  return launch_jit(A, fn, args, (rows + rpb - 1) / rpb, stream, "row_reduce");
}

// Chain + reduction over every element; n must be a whole number of units of E elements.
int launch_full_reduce_jit(const void* const* in, void* out, float* partials, unsigned int* ticket, const int* in_dt,
                           int out_dt, const cdr_ew_params& p, int reduce_op, int64_t n_units, int64_t cols, int E,
                           int grid, cudaStream_t stream) {
  const Api& A = api();
  if (!A.ok) return CDR_ERR_UNSUPPORTED;
  CUfunction fn = nullptr;
  if (int rc = get_kernel(A, generate_full_reduce(p, in_dt, out_dt, reduce_op, E, E == 4 ? 4 : 2), &fn)) return rc;
  JitArgs args{};
  for (int i = 0; i < p.n_inputs; ++i) args.in[i] = in[i];
  args.out[0] = out;
  args.out[1] = partials;
  args.out[2] = ticket;
  args.n_units = n_units;
  args.cols = cols;
  return launch_jit(A, fn, args, grid, stream, "full_reduce");
}

}  // namespace cdr
