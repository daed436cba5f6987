// C ABI of libconductor_b200.so: argument checking, template dispatch, the
// host-pointer entry point and its per-device staging arena.
//
// Replaces the C++ wrapper the reference generates per compiled graph
// (conductor/compiler/host_wrapper.py:108-197).  No exception leaves this file.
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <mutex>
#include <new>
#include <vector>

#include <string>

#include "cdr_common.cuh"

namespace cdr {

std::string jit_elementwise_source(const cdr_ew_params& p, const int* in_dt, const int* out_dt, int E);
std::string jit_row_reduce_source(const cdr_ew_params& p, const int* in_dt, int out_dt, int reduce_op, int E, int64_t cols);
std::string jit_full_reduce_source(const cdr_ew_params& p, const int* in_dt, int out_dt, int reduce_op, int E);
std::vector<char> jit_compile(const std::string& src, std::string* log);
int validate_ew_program(const cdr_ew_params* p, int n_in, int n_out);

namespace {
thread_local char g_error[512] = {0};
constexpr int kMaxDevices = 64;
int g_sm_count[kMaxDevices] = {0};
}  // namespace

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

int cuda_fail(cudaError_t e, const char* what) {
  set_error("CUDA error %d (%s) in %s", static_cast<int>(e), cudaGetErrorString(e), what);
  return CDR_ERR_CUDA;
}

// One status word per device; kernels get its address as an argument.
__device__ int g_status_word = 0;
namespace {
int* g_status_ptr[64] = {nullptr};
}
int* device_status_ptr() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!g_status_ptr[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) return nullptr;
    g_status_ptr[dev] = static_cast<int*>(p);
  }
  return g_status_ptr[dev];
}

int sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
  if (g_sm_count[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    g_sm_count[dev] = n;  // benign race: every writer stores the same value
  }
  return g_sm_count[dev];
}

void clear_error() { g_error[0] = 0; }

int check_lists(const cdr_tensor* ins, int n_in, const cdr_tensor* outs, int n_out) {
  if (n_in < 0 || n_out < 0 || (n_in > 0 && !ins) || (n_out > 0 && !outs)) {
    set_error("tensor list is null or has a negative count");
    return CDR_ERR_BAD_ARG;
  }
  for (int pass = 0; pass < 2; ++pass) {
    const cdr_tensor* t = pass ? outs : ins;
    const int n = pass ? n_out : n_in;
    for (int i = 0; i < n; ++i) {
      if (t[i].rank < 0 || t[i].rank > CDR_MAX_RANK) {
        set_error("%s %d has rank %d (max %d)", pass ? "output" : "input", i, t[i].rank, CDR_MAX_RANK);
        return CDR_ERR_BAD_ARG;
      }
      if (dtype_size(t[i].dtype) == 0) {
        set_error("%s %d has unknown dtype %d", pass ? "output" : "input", i, t[i].dtype);
        return CDR_ERR_BAD_ARG;
      }
      for (int d = 0; d < t[i].rank; ++d)
        if (t[i].shape[d] < 0) {
          set_error("%s %d has a negative extent", pass ? "output" : "input", i);
          return CDR_ERR_BAD_ARG;
        }
    }
  }
  return CDR_OK;
}

namespace {

int check_params(int template_id, const void* params, size_t bytes) {
  size_t want = 0;
  switch (template_id) {
    case CDR_T_ELEMENTWISE: want = sizeof(cdr_ew_params); break;
    case CDR_T_ROW_REDUCE:
    case CDR_T_FULL_REDUCE: want = sizeof(cdr_reduce_params); break;
    case CDR_T_SOFTMAX_FWD:
    case CDR_T_SOFTMAX_BWD:
    case CDR_T_COL_SUM:
    case CDR_T_COPY: return CDR_OK;
    case CDR_T_GEMM_EPILOGUE: want = sizeof(cdr_gemm_params); break;
    case CDR_T_ATTENTION: want = sizeof(cdr_attn_params); break;
    case CDR_T_LAYER_NORM: want = sizeof(cdr_norm_params); break;
    default:
      set_error("unknown template id %d", template_id);
      return CDR_ERR_UNSUPPORTED;
  }
  if (!params || bytes != want) {
    set_error("template %d expects a %zu-byte parameter block, got %zu", template_id, want, params ? bytes : (size_t)0);
    return CDR_ERR_BAD_ARG;
  }
  return CDR_OK;
}

// ---- staging arena for cdr_execute_host: one growing device buffer per device ----
struct Arena {
  void* base = nullptr;
  size_t bytes = 0;
  cudaStream_t stream = nullptr;
};
std::mutex g_arena_mu;
Arena g_arena[kMaxDevices];

size_t round256(size_t n) { return (n + 255) & ~static_cast<size_t>(255); }

}  // namespace
}  // namespace cdr

using namespace cdr;

extern "C" {

int cdr_abi_version(void) { return CDR_ABI_VERSION; }

const char* cdr_status_string(int status) {
  switch (status) {
    case CDR_OK: return "ok";
    case CDR_ERR_BAD_ARG: return "bad argument";
    case CDR_ERR_UNSUPPORTED: return "unsupported by this kernel template";
    case CDR_ERR_MISALIGNED: return "misaligned pointer";
    case CDR_ERR_CUDA: return "CUDA runtime error";
    case CDR_ERR_TIMEOUT: return "device-side wait timed out";
    case CDR_ERR_WORKSPACE: return "workspace missing or too small";
    default: return "unknown status";
  }
}

const char* cdr_last_error(void) { return g_error; }

int cdr_device_count(void) {
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDeviceCount");
  return n;
}

int cdr_device_status(int* status_out, int clear) {
  if (!status_out) { set_error("status_out is null"); return CDR_ERR_BAD_ARG; }
  *status_out = 0;
  int* p = device_status_ptr();
  if (!p) { set_error("device status word unavailable"); return CDR_ERR_CUDA; }
  CDR_CUDA_TRY(cudaDeviceSynchronize());
  CDR_CUDA_TRY(cudaMemcpy(status_out, p, sizeof(int), cudaMemcpyDeviceToHost));
  if (clear && *status_out) CDR_CUDA_TRY(cudaMemset(p, 0, sizeof(int)));
  return *status_out ? CDR_ERR_TIMEOUT : CDR_OK;
}

int cdr_template_source(int template_id, const cdr_tensor* inputs, int n_inputs, const cdr_tensor* outputs, int n_outputs,
                        const void* params, size_t params_bytes, char* buffer, size_t buffer_bytes, int compile) {
  g_error[0] = 0;
  if (template_id != CDR_T_ELEMENTWISE && template_id != CDR_T_ROW_REDUCE && template_id != CDR_T_FULL_REDUCE) {
    set_error("template %d has no run-time instances", template_id);
    return CDR_ERR_UNSUPPORTED;
  }
  if (int rc = check_lists(inputs, n_inputs, outputs, n_outputs)) return rc;
  if (int rc = check_params(template_id, params, params_bytes)) return rc;
  const bool reduce = template_id != CDR_T_ELEMENTWISE;
  const cdr_ew_params* p = reduce ? &static_cast<const cdr_reduce_params*>(params)->chain : static_cast<const cdr_ew_params*>(params);
  if (int rc = validate_ew_program(p, n_inputs, n_outputs)) return rc;
  if (reduce && (n_outputs != 1 || n_inputs < 1)) { set_error("row_reduce: needs >=1 input and exactly one output"); return CDR_ERR_BAD_ARG; }
  if (!buffer || buffer_bytes == 0) { set_error("buffer is null or empty"); return CDR_ERR_BAD_ARG; }
  int in_dt[CDR_EW_MAX_INPUTS] = {0}, out_dt[CDR_EW_MAX_OUTPUTS] = {0};
  bool any16 = false;
  for (int i = 0; i < n_inputs; ++i) { in_dt[i] = inputs[i].dtype; any16 |= dtype_size(in_dt[i]) == 2; }
  for (int o = 0; o < n_outputs; ++o) { out_dt[o] = outputs[o].dtype; if (!reduce) any16 |= dtype_size(out_dt[o]) == 2; }
  for (int i = 0; i < n_inputs + n_outputs; ++i) {
    const int dt = i < n_inputs ? in_dt[i] : out_dt[i - n_inputs];
    const bool flag_ok = dt == CDR_BOOL && !reduce;   // bool masks and bool results: elementwise only
    if (dt != CDR_F32 && dt != CDR_BF16 && dt != CDR_F16 && !flag_ok) { set_error("only floating-point programs (with bool operands in elementwise ones) are instantiated at run time"); return CDR_ERR_UNSUPPORTED; }
  }
  std::string src;
  try {
    if (reduce) {
      int64_t cols = 0;
      for (int i = 0; i < n_inputs; ++i)
        if (p->input_mode[i] == CDR_IN_FULL && inputs[i].rank >= 1) { cols = inputs[i].shape[inputs[i].rank - 1]; break; }
      const int rop = static_cast<const cdr_reduce_params*>(params)->reduce_op;
      src = template_id == CDR_T_FULL_REDUCE ? jit_full_reduce_source(*p, in_dt, out_dt[0], rop, any16 ? 8 : 4)
                                             : jit_row_reduce_source(*p, in_dt, out_dt[0], rop, any16 ? 8 : 4, cols);
    } else {
      src = jit_elementwise_source(*p, in_dt, out_dt, any16 ? 8 : 4);
    }
    const size_t n = src.size() < buffer_bytes - 1 ? src.size() : buffer_bytes - 1;
    memcpy(buffer, src.data(), n);
    buffer[n] = 0;
    if (compile) {
      std::string log;
      if (jit_compile(src, &log).empty()) {
        set_error("NVRTC: %s", log.empty() ? "compilation failed" : log.c_str());
        return CDR_ERR_UNSUPPORTED;
      }
    }
  } catch (const std::exception& e) {
    set_error("source generation failed: %s", e.what());
    return CDR_ERR_BAD_ARG;
  }
  return CDR_OK;
}

int cdr_workspace_bytes(int template_id, const cdr_tensor* inputs, int n_inputs, const cdr_tensor* outputs,
                        int n_outputs, const void* params, size_t params_bytes, size_t* bytes_out) {
  if (!bytes_out) { set_error("bytes_out is null"); return CDR_ERR_BAD_ARG; }
  *bytes_out = 0;
  if (int rc = check_lists(inputs, n_inputs, outputs, n_outputs)) return rc;
  if (int rc = check_params(template_id, params, params_bytes)) return rc;
  switch (template_id) {
    case CDR_T_FULL_REDUCE: return full_reduce_workspace(inputs, n_inputs, bytes_out);
    case CDR_T_ATTENTION: return attention_workspace(inputs, n_inputs, bytes_out);
    case CDR_T_COL_SUM: return col_sum_workspace(inputs, n_inputs, outputs, n_outputs, bytes_out);
    default: return CDR_OK;
  }
}

int cdr_launch(int template_id, const cdr_tensor* inputs, int n_inputs, const cdr_tensor* outputs, int n_outputs,
               const void* params, size_t params_bytes, void* workspace, size_t workspace_bytes, void* cuda_stream) {
  g_error[0] = 0;
  if (int rc = check_lists(inputs, n_inputs, outputs, n_outputs)) return rc;
  if (int rc = check_params(template_id, params, params_bytes)) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
  switch (template_id) {
    case CDR_T_ELEMENTWISE:
      return launch_elementwise(inputs, n_inputs, outputs, n_outputs, static_cast<const cdr_ew_params*>(params), s);
    case CDR_T_ROW_REDUCE:
      return launch_row_reduce(inputs, n_inputs, outputs, n_outputs, static_cast<const cdr_reduce_params*>(params), s);
    case CDR_T_FULL_REDUCE:
      return launch_full_reduce(inputs, n_inputs, outputs, n_outputs, static_cast<const cdr_reduce_params*>(params),
                                workspace, workspace_bytes, s);
    case CDR_T_SOFTMAX_FWD: return launch_softmax_fwd(inputs, n_inputs, outputs, n_outputs, s);
    case CDR_T_SOFTMAX_BWD: return launch_softmax_bwd(inputs, n_inputs, outputs, n_outputs, s);
    case CDR_T_GEMM_EPILOGUE:
      return launch_gemm_epilogue(inputs, n_inputs, outputs, n_outputs, static_cast<const cdr_gemm_params*>(params), s);
    case CDR_T_ATTENTION:
      return launch_attention(inputs, n_inputs, outputs, n_outputs, static_cast<const cdr_attn_params*>(params),
                              workspace, workspace_bytes, s);
    case CDR_T_COPY: return launch_strided_copy(inputs, n_inputs, outputs, n_outputs, s);
    case CDR_T_COL_SUM: return launch_col_sum(inputs, n_inputs, outputs, n_outputs, workspace, workspace_bytes, s);
    case CDR_T_LAYER_NORM:
      return launch_layer_norm(inputs, n_inputs, outputs, n_outputs, static_cast<const cdr_norm_params*>(params), s);
    default:
      set_error("unknown template id %d", template_id);
      return CDR_ERR_UNSUPPORTED;
  }
}

int cdr_launch_many(const cdr_launch_item* items, int n_items, void* cuda_stream, int* failed_item) {
  g_error[0] = 0;
  if (failed_item) *failed_item = -1;
  if (n_items < 0 || (n_items > 0 && !items)) { set_error("launch list is null or has a negative count"); return CDR_ERR_BAD_ARG; }
  for (int i = 0; i < n_items; ++i) {
    const cdr_launch_item& it = items[i];
    const int rc = cdr_launch(it.template_id, it.inputs, it.n_inputs, it.outputs, it.n_outputs, it.params, it.params_bytes,
                              it.workspace, it.workspace_bytes, cuda_stream);
    if (rc != CDR_OK) {
      if (failed_item) *failed_item = i;
      return rc;
    }
  }
  return CDR_OK;
}

int cdr_execute_host(int template_id, const cdr_tensor* host_inputs, int n_inputs, const cdr_tensor* host_outputs,
                     int n_outputs, const void* params, size_t params_bytes, int device) {
  g_error[0] = 0;
  if (int rc = check_lists(host_inputs, n_inputs, host_outputs, n_outputs)) return rc;
  if (int rc = check_params(template_id, params, params_bytes)) return rc;
  if (device < 0 || device >= kMaxDevices) { set_error("device %d out of range", device); return CDR_ERR_BAD_ARG; }
  CDR_CUDA_TRY(cudaSetDevice(device));

  size_t ws_bytes = 0;
  if (int rc = cdr_workspace_bytes(template_id, host_inputs, n_inputs, host_outputs, n_outputs, params, params_bytes,
                                   &ws_bytes))
    return rc;

  std::vector<cdr_tensor> din, dout;
  std::vector<size_t> off;
  size_t total = 0;
  try {
    din.assign(host_inputs, host_inputs + n_inputs);
    dout.assign(host_outputs, host_outputs + n_outputs);
    off.reserve(static_cast<size_t>(n_inputs + n_outputs) + 1);
  } catch (const std::bad_alloc&) {
    set_error("out of host memory");
    return CDR_ERR_BAD_ARG;
  }
  for (int i = 0; i < n_inputs; ++i) {
    if (!is_contiguous(din[i])) { set_error("host input %d is not contiguous", i); return CDR_ERR_BAD_ARG; }
    off.push_back(total);
    total += round256(static_cast<size_t>(numel(din[i])) * dtype_size(din[i].dtype));
  }
  for (int i = 0; i < n_outputs; ++i) {
    if (!is_contiguous(dout[i])) { set_error("host output %d is not contiguous", i); return CDR_ERR_BAD_ARG; }
    off.push_back(total);
    total += round256(static_cast<size_t>(numel(dout[i])) * dtype_size(dout[i].dtype));
  }
  const size_t ws_off = total;
  total += round256(ws_bytes);

  // One call at a time per process on the host path: the arena is shared state.
  std::lock_guard<std::mutex> lock(g_arena_mu);
  Arena& ar = g_arena[device];
  if (!ar.stream) CDR_CUDA_TRY(cudaStreamCreateWithFlags(&ar.stream, cudaStreamNonBlocking));
  if (ar.bytes < total) {
    if (ar.base) { CDR_CUDA_TRY(cudaFree(ar.base)); ar.base = nullptr; ar.bytes = 0; }
    CDR_CUDA_TRY(cudaMalloc(&ar.base, total));
    ar.bytes = total;
  }
  char* base = static_cast<char*>(ar.base);
  for (int i = 0; i < n_inputs; ++i) {
    const size_t nb = static_cast<size_t>(numel(din[i])) * dtype_size(din[i].dtype);
    if (nb && !host_inputs[i].data) { set_error("host input %d has a null pointer", i); return CDR_ERR_BAD_ARG; }
    din[i].data = base + off[i];
    if (nb) CDR_CUDA_TRY(cudaMemcpyAsync(din[i].data, host_inputs[i].data, nb, cudaMemcpyHostToDevice, ar.stream));
  }
  for (int i = 0; i < n_outputs; ++i) dout[i].data = base + off[n_inputs + i];

  int rc = cdr_launch(template_id, din.data(), n_inputs, dout.data(), n_outputs, params, params_bytes,
                      ws_bytes ? base + ws_off : nullptr, ws_bytes, ar.stream);
  if (rc != CDR_OK) {
    cudaStreamSynchronize(ar.stream);
    return rc;
  }
  for (int i = 0; i < n_outputs; ++i) {
    const size_t nb = static_cast<size_t>(numel(dout[i])) * dtype_size(dout[i].dtype);
    if (nb && !host_outputs[i].data) { set_error("host output %d has a null pointer", i); cudaStreamSynchronize(ar.stream); return CDR_ERR_BAD_ARG; }
    if (nb) CDR_CUDA_TRY(cudaMemcpyAsync(host_outputs[i].data, dout[i].data, nb, cudaMemcpyDeviceToHost, ar.stream));
  }
  CDR_CUDA_TRY(cudaStreamSynchronize(ar.stream));
  return CDR_OK;
}

int cdr_release_host_arena(int device) {
  std::lock_guard<std::mutex> lock(g_arena_mu);
  int prev = 0;
  const bool have_prev = cudaGetDevice(&prev) == cudaSuccess;
  for (int d = 0; d < kMaxDevices; ++d) {
    if (device >= 0 && d != device) continue;
    Arena& ar = g_arena[d];
    if (!ar.base && !ar.stream) continue;
    if (cudaSetDevice(d) != cudaSuccess) continue;
    if (ar.base) cudaFree(ar.base);
    if (ar.stream) cudaStreamDestroy(ar.stream);
    ar = Arena{};
  }
  if (have_prev) cudaSetDevice(prev);
  return CDR_OK;
}

}  // extern "C"
