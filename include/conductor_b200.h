/*
 * conductor_b200.h -- C ABI of libconductor_b200.so
 *
 * One prebuilt shared library replaces the per-graph C++ host wrapper that the
 * reference backend generates, compiles and dlopens for every compiled graph
 * (reference: conductor/compiler/host_wrapper.py:108-197, the emitted
 * `extern "C" int execute_kernel(void* input_data_0, size_t* input_shape_0, ...,
 * void* output_data, size_t* output_shape)`; loaded with ctypes at
 * host_wrapper.py:338-355 and called at host_wrapper.py:360-403).
 *
 * Conventions kept from that interface:
 *   - C linkage, `int` status return, 0 = success, non-zero = failure
 *     (host_wrapper.py:186-194: 0 / -1 / -2); no C++ exception crosses the boundary.
 *   - The caller owns every buffer, inputs and outputs alike
 *     (conductor/compiler/executor.py:611); the library keeps no pointer after a call.
 *   - Tensors are contiguous row-major (host_wrapper.py:380-392).
 *
 * Differences, all forced by running on a GPU:
 *   - cdr_launch() takes DEVICE pointers and a CUDA stream and is asynchronous.
 *   - cdr_execute_host() keeps the reference's synchronous host-pointer contract
 *     (the generated wrapper copies host->device, runs, copies back:
 *     host_wrapper.py:169-182).
 *   - A fused cluster is named by a template id plus a small parameter block
 *     instead of by a generated symbol name.
 *
 * Every kernel behind this ABI is compiled for sm_100a only.  There is no CPU
 * implementation in the library: without a usable CUDA device every compute
 * entry point returns CDR_ERR_CUDA.
 */
#ifndef CONDUCTOR_B200_H_
#define CONDUCTOR_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define CDR_API __attribute__((visibility("default")))
#else
#define CDR_API
#endif

#define CDR_ABI_VERSION 1
#define CDR_MAX_RANK 8

/* ---- status codes (reference: host_wrapper.py:186-194 returns 0/-1/-2; Python raises
 * ExecutionError on non-zero at executor.py:621-622) ---- */
enum cdr_status {
  CDR_OK = 0,
  CDR_ERR_BAD_ARG = -1,     /* null pointer, wrong tensor count, shape mismatch        */
  CDR_ERR_UNSUPPORTED = -2, /* dtype / shape / program the template cannot run         */
  CDR_ERR_MISALIGNED = -3,  /* a pointer violates the template's alignment requirement */
  CDR_ERR_CUDA = -4,        /* a CUDA runtime call failed; see cdr_last_error()        */
  CDR_ERR_TIMEOUT = -5,     /* a bounded device-side wait gave up                      */
  CDR_ERR_WORKSPACE = -6    /* workspace missing or smaller than cdr_workspace_bytes() */
};

/* ---- element types (reference dtype table: host_wrapper.py:50-56 plus bf16 from
 * conductor/utils/type_mapping.py:76-91) ---- */
enum cdr_dtype {
  CDR_F32 = 0,
  CDR_BF16 = 1,
  CDR_F16 = 2,
  CDR_I32 = 3,
  CDR_I64 = 4,
  CDR_BOOL = 5
};

/* ---- tensor descriptor: replaces the (void* data, size_t* shape) pairs of the
 * reference wrapper (host_wrapper.py:132-145) and choreo.h's spanned_view
 * (choreo-headers/choreo.h:604-662).  Strides are in elements. ---- */
typedef struct cdr_tensor {
  void* data;
  int32_t dtype; /* enum cdr_dtype */
  int32_t rank;
  int64_t shape[CDR_MAX_RANK];
  int64_t stride[CDR_MAX_RANK];
} cdr_tensor;

/* ---- fused-cluster templates.  One id per cluster kind the fusion engine emits
 * (reference cluster kinds: conductor/optimization/fusion.py:30-38). ---- */
enum cdr_template {
  CDR_T_ELEMENTWISE = 1,  /* chain of elementwise ops, params = cdr_ew_params            */
  CDR_T_ROW_REDUCE = 2,   /* elementwise chain + reduction over the last dim,
                             params = cdr_reduce_params                                  */
  CDR_T_SOFTMAX_FWD = 3,  /* row softmax over the last dim, no params                    */
  CDR_T_SOFTMAX_BWD = 4,  /* inputs (grad_out, y): dx = y * (g - sum(g*y)), no params    */
  CDR_T_GEMM_EPILOGUE = 5,/* out = act(x @ W^T + bias) or act(x @ W + bias), params = cdr_gemm_params */
  CDR_T_ATTENTION = 6,    /* fused scaled-dot-product attention, params = cdr_attn_params*/
  CDR_T_FULL_REDUCE = 7,  /* elementwise chain + reduction over every element,
                             params = cdr_reduce_params; needs workspace                 */
  CDR_T_LAYER_NORM = 8,   /* layer normalisation over the last dim, inputs (x[, weight][, bias]),
                             params = cdr_norm_params                                    */
  CDR_T_COPY = 9,         /* copy a strided view (the input descriptor's strides are honoured; stride 0
                             broadcasts) into an output of the same shape: transpose / permute / slice /
                             expand / contiguous().  The output's strides are honoured too (positive,
                             non-overlapping), which writes one part of a concatenation; no params */
  CDR_T_COL_SUM = 10      /* out[n] = sum over m of x[m, n] for a contiguous x viewed as [M, N] (N = the
                             output's element count): the bias gradient of a linear layer, `sum(dim=0)`.
                             fp32 accumulation in a fixed order (deterministic); no params; needs workspace.
                             The reference has no counterpart: it compiles no backward graphs */
};

/* ---- elementwise programs -------------------------------------------------
 * A chain is a straight-line program over virtual registers.  Registers
 * 0..n_inputs-1 hold the cluster's external inputs (converted to fp32, or kept
 * as int64 for integer tensors); instruction i writes register n_inputs+i.
 * After each instruction the value is rounded to `round_to` when that is
 * CDR_BF16/CDR_F16, which reproduces eager execution of a low-precision graph
 * op by op (the reference's executed path, conductor/compiler/gcu_backend.py:89).
 */
enum cdr_ew_op {
  CDR_OP_ADD = 1,      /* r[a] + r[b]                   */
  CDR_OP_SUB = 2,      /* r[a] - r[b]                   */
  CDR_OP_MUL = 3,      /* r[a] * r[b]                   */
  CDR_OP_DIV = 4,      /* r[a] / r[b]                   */
  CDR_OP_RELU = 5,     /* max(r[a], 0), NaN propagates  */
  CDR_OP_NEG = 6,
  CDR_OP_ABS = 7,
  CDR_OP_EXP = 8,
  CDR_OP_LOG = 9,
  CDR_OP_SQRT = 10,
  CDR_OP_SIGMOID = 11,
  CDR_OP_TANH = 12,
  CDR_OP_SIN = 13,
  CDR_OP_COS = 14,
  CDR_OP_MAX = 15,     /* max(r[a], r[b])               */
  CDR_OP_MIN = 16,
  CDR_OP_ADDCDIV = 17, /* r[a] + (imm * r[b]) / r[c]    */
  CDR_OP_ADDCMUL = 18, /* r[a] + (imm * r[b]) * r[c]    */
  CDR_OP_CONST = 19,   /* imm                           */
  CDR_OP_COPY = 20,    /* r[a] (used for dtype casts: only the rounding applies) */
  CDR_OP_ADD_IMM = 21, /* r[a] + imm                    */
  CDR_OP_MUL_IMM = 22, /* r[a] * imm                    */
  CDR_OP_RSUB_IMM = 23,/* imm - r[a]                    */
  CDR_OP_RDIV_IMM = 24,/* imm / r[a]                    */
  CDR_OP_GT = 25,      /* r[a] >  r[b] ? 1 : 0 (comparisons yield 1.0 / 0.0; NaN compares false, NE true) */
  CDR_OP_GE = 26,
  CDR_OP_LT = 27,
  CDR_OP_LE = 28,
  CDR_OP_EQ = 29,
  CDR_OP_NE = 30,
  CDR_OP_WHERE = 31,   /* r[a] != 0 ? r[b] : r[c]       */
  CDR_OP_RSQRT = 32,   /* 1 / sqrt(r[a])                */
  CDR_OP_SILU = 33,    /* r[a] / (1 + exp(-r[a]))       */
  CDR_OP_GELU = 34,    /* 0.5 r[a] (1 + erf(r[a] / sqrt 2)) */
  CDR_OP_ERF = 35
};
#define CDR_OP_LAST CDR_OP_ERF

/* how an external input is indexed against the [rows, cols] view of the output */
enum cdr_ew_mode {
  CDR_IN_FULL = 0,   /* same shape as the output                       */
  CDR_IN_ROW = 1,    /* shape [cols], broadcast over rows              */
  CDR_IN_COL = 2,    /* shape [rows, 1], broadcast over columns        */
  CDR_IN_SCALAR = 3  /* one element                                    */
};

#define CDR_EW_MAX_INPUTS 8
#define CDR_EW_MAX_INSTR 24
#define CDR_EW_MAX_OUTPUTS 4

typedef struct cdr_ew_instr {
  int32_t op;       /* enum cdr_ew_op                                  */
  int32_t a, b, c;  /* source registers (unused ones are 0)            */
  float imm;        /* immediate for *_IMM / CONST / ADDCDIV / ADDCMUL */
  int32_t round_to; /* enum cdr_dtype of the op's result               */
} cdr_ew_instr;

typedef struct cdr_ew_params {
  int32_t n_inputs;
  int32_t n_instr;
  int32_t n_outputs;
  int32_t reserved;
  int32_t input_mode[CDR_EW_MAX_INPUTS]; /* enum cdr_ew_mode per input        */
  int32_t out_reg[CDR_EW_MAX_OUTPUTS];   /* register stored to each output    */
  cdr_ew_instr instr[CDR_EW_MAX_INSTR];
} cdr_ew_params;

enum cdr_reduce_op { CDR_RED_SUM = 1, CDR_RED_MEAN = 2, CDR_RED_MAX = 3, CDR_RED_MIN = 4 };

typedef struct cdr_reduce_params {
  cdr_ew_params chain; /* chain.out_reg[0] is the value that is reduced; n_outputs = 1 */
  int32_t reduce_op;   /* enum cdr_reduce_op                                           */
  int32_t reserved;
} cdr_reduce_params;

enum cdr_activation { CDR_ACT_NONE = 0, CDR_ACT_RELU = 1 };

enum cdr_weight_layout {
  CDR_W_NK = 0, /* W is [N, K], K contiguous: out = x @ W^T  (torch.nn.functional.linear) */
  CDR_W_KN = 1  /* W is [K, N], N contiguous: out = x @ W    (torch.matmul)               */
};

enum cdr_x_layout {
  CDR_X_MK = 0, /* x is [..., K], K contiguous                                            */
  CDR_X_KM = 1  /* x is [K, M], M contiguous: out = x^T @ ...  (weight gradients)          */
};

typedef struct cdr_gemm_params {
  int32_t activation;    /* enum cdr_activation                       */
  int32_t has_bias;      /* 1: inputs are (x, W, bias); 0: (x, W)     */
  int32_t weight_layout; /* enum cdr_weight_layout                    */
  int32_t x_layout;      /* enum cdr_x_layout                         */
  int32_t gate_input;    /* 1: the LAST input is a tensor shaped like the output whose positive entries let the
                            result through and whose other entries zero it: out = (gate > 0) ? result : 0.
                            The backward of a ReLU fused into the product that makes its incoming gradient
                            (dZ = (dY @ W) * (H > 0)).  The reference has no counterpart (no backward graphs) */
} cdr_gemm_params;

typedef struct cdr_norm_params {
  float eps;
  int32_t has_weight; /* 1: a [cols] scale follows x in the inputs           */
  int32_t has_bias;   /* 1: a [cols] shift is the last input                 */
  int32_t reserved;
} cdr_norm_params;

typedef struct cdr_attn_params {
  float scale;    /* softmax scale, e.g. 1/sqrt(head_dim) */
  int32_t causal; /* 1: key j attends only when j <= i    */
} cdr_attn_params;

/* ---- entry points --------------------------------------------------------- */

/* ABI version of the loaded library (== CDR_ABI_VERSION of the header it was built
 * from).  No counterpart in the reference; lets a binding reject a stale .so. */
CDR_API int cdr_abi_version(void);

/* Static, human-readable name of a status code.  Replaces the std::cerr text the
 * reference wrapper prints before returning -1/-2 (host_wrapper.py:186-194). */
CDR_API const char* cdr_status_string(int status);

/* Message of the last failure on the calling thread (empty string if none).
 * Replaces the reference wrapper's std::cerr diagnostics (host_wrapper.py:188,192). */
CDR_API const char* cdr_last_error(void);

/* Number of CUDA devices visible to the library, or a negative cdr_status.
 * Replaces the device probe in conductor/compiler/topscc_utils.py:27-29. */
CDR_API int cdr_device_count(void);

/* Wait for the current device and read its status word: kernels whose bounded device-side
 * waits gave up record (1 << 8 | site) there.  Returns CDR_OK (word is 0) or CDR_ERR_TIMEOUT
 * with the word in *status_out; `clear` != 0 resets it.  Replaces the device-side
 * `future` misuse detection of the reference runtime header (choreo-headers/choreo.h:1013-1112). */
CDR_API int cdr_device_status(int* status_out, int clear);

/* CUDA source of the kernel instance an elementwise or row-reduce program runs when it has no
 * ahead-of-time instance (the hand-written streaming skeleton specialised with the program),
 * written NUL-terminated into `buffer` (truncated to buffer_bytes).  With `compile` != 0 the source
 * is also compiled for sm_100a with NVRTC -- no GPU needed -- and CDR_ERR_UNSUPPORTED is returned
 * with the compiler log in cdr_last_error() if that fails.  Only dtypes, the last dimension and the
 * program are read from the descriptors.  template_id is CDR_T_ELEMENTWISE, CDR_T_ROW_REDUCE or
 * CDR_T_FULL_REDUCE.
 * Replaces the generated-DSL dump of the reference
 * (conductor/codegen/dslgen.py:154-177 generate_dsl_file, conductor/utils/artifacts.py:18-237). */
CDR_API int cdr_template_source(int template_id, const cdr_tensor* inputs, int n_inputs, const cdr_tensor* outputs,
                                int n_outputs, const void* params, size_t params_bytes, char* buffer,
                                size_t buffer_bytes, int compile);

/* Bytes of device workspace cdr_launch() needs for this call (0 for most
 * templates).  Replaces the fixed `memory_pool_size_mb` of the reference runtime
 * configuration (conductor/utils/config.py:66-72). */
CDR_API int cdr_workspace_bytes(int template_id, const cdr_tensor* inputs, int n_inputs,
                        const cdr_tensor* outputs, int n_outputs, const void* params,
                        size_t params_bytes, size_t* bytes_out);

/* Run one fused cluster on device-resident tensors, asynchronously on `cuda_stream`
 * (a cudaStream_t; NULL = the legacy default stream) of the current device.
 * Replaces execute_kernel() (host_wrapper.py:132-196) as called from
 * ChoreoHostInterface.execute_kernel_with_library (host_wrapper.py:360-403). */
CDR_API int cdr_launch(int template_id, const cdr_tensor* inputs, int n_inputs,
               const cdr_tensor* outputs, int n_outputs, const void* params,
               size_t params_bytes, void* workspace, size_t workspace_bytes,
               void* cuda_stream);

/* One step of a plan for cdr_launch_many(): the arguments of one cdr_launch() call. */
typedef struct cdr_launch_item {
  int32_t template_id;
  int32_t n_inputs;
  int32_t n_outputs;
  int32_t reserved;            /* 0 */
  const cdr_tensor* inputs;
  const cdr_tensor* outputs;
  const void* params;
  size_t params_bytes;
  void* workspace;
  size_t workspace_bytes;
} cdr_launch_item;

/* Run the steps of a compiled plan in order on one stream with a single call.  The reference's
 * generated execute_kernel() runs a whole compiled graph per call (host_wrapper.py:132-196); a
 * plan here may hold several clusters, and crossing the FFI once per plan instead of once per
 * cluster keeps short plans from being bound by host time.  Equivalent to calling cdr_launch()
 * per item: stops at the first failing item, returns its status and stores its index in
 * *failed_item (when not NULL).  Buffers that one item writes and a later item reads are ordered
 * by the stream. */
CDR_API int cdr_launch_many(const cdr_launch_item* items, int n_items, void* cuda_stream, int* failed_item);

/* Same cluster, reference calling convention: HOST pointers in, HOST pointers out,
 * synchronous.  Copies inputs to `device`, launches, copies outputs back and waits
 * (host_wrapper.py:169-182).  Staging memory is a per-device arena owned by the
 * library and grown on demand; cdr_release_host_arena() frees it. */
CDR_API int cdr_execute_host(int template_id, const cdr_tensor* host_inputs, int n_inputs,
                     const cdr_tensor* host_outputs, int n_outputs, const void* params,
                     size_t params_bytes, int device);

/* Free the staging arena cdr_execute_host() grew on `device` (-1: every device).
 * Replaces GCUKernelExecutor.unload_kernel (conductor/compiler/executor.py:64-90). */
CDR_API int cdr_release_host_arena(int device);

/* CDR_T_FULL_REDUCE without a caller workspace and without any allocation.  (No counterpart
 * in the reference: it has no allocation-free calling mode.)
 *
 * For hosts that cannot call cudaMalloc while running: servers or framework pools that
 * reserved all device memory up front, and loops that cannot afford the device-wide
 * synchronisation an allocation brings.  The scratch the reduction needs (a ticket counter and
 * one fp32 partial per CTA) is a fixed array inside the library's device image: 4352 bytes =
 * 256 + 4 * 1024 partial sums, resident on every GPU that loads the library until exit.  The
 * reduction runs 4 CTAs per SM, so devices with up to 256 SMs fit; otherwise the call returns
 * CDR_ERR_UNSUPPORTED and cdr_last_error() names the needed and available sizes.
 *
 * inputs / outputs / params are exactly those of cdr_launch(CDR_T_FULL_REDUCE, ...); the
 * caller still owns them.  The call always runs the kernel compiled into the library: it never
 * takes the run-time-instance path of cdr_launch (whose first use per program compiles with NVRTC
 * and loads a module, which allocates device memory), so results may differ from cdr_launch's by
 * fp32 summation order.  The first call on a device resolves the array's device address and
 * should therefore be made before any stream capture begins.  Every call on a device shares the
 * one array: the ticket is cleared at the start of each call, and calls whose kernels could
 * overlap on the GPU (different streams without ordering) race and must be serialised. */
CDR_API int cdr_full_reduce_noalloc(const cdr_tensor* inputs, int n_inputs, const cdr_tensor* outputs,
                                    int n_outputs, const void* params, size_t params_bytes,
                                    void* cuda_stream);

#ifdef __cplusplus
}
#endif
#endif /* CONDUCTOR_B200_H_ */
