// K7 -- strided copy: the materialising form of transpose / permute / slicing / expand /
// .contiguous() on a view, and (with a strided output) the scatter of one part into a
// concatenation.
//
// The reference forces every kernel operand contiguous on the host before a call
// (conductor/compiler/host_wrapper.py:380-392, `tensor.contiguous()`); here the copy is a template
// of its own so that a permuted view never has to leave the device path.  The input descriptor
// carries the view's shape and element strides; the output has the same shape and is normally
// contiguous, but may itself be a strided view (non-overlapping; the caller's responsibility) --
// `cat` writes each part into its slice of the result that way.
// HBM-bound.  When the view's innermost dimension is contiguous in memory and a whole number of
// 16-byte vectors (the head-dimension case: [B, S, H, D] -> [B, H, S, D]), every thread moves one
// 16-byte vector with streaming accesses; otherwise elements are gathered one by one (reads
// uncoalesced when the innermost stride is not 1).
#include "cdr_common.cuh"

namespace cdr {
namespace {

struct CopyArgs {
  const unsigned char* in;
  unsigned char* out;
  int64_t n_units;              // units of `unit_bytes`
  int32_t rank;
  int32_t unit_bytes;           // 16 on the vector path, the element size otherwise
  int64_t shape[CDR_MAX_RANK];  // output shape in units (innermost dimension divided on the vector path)
  int64_t stride[CDR_MAX_RANK]; // input strides in bytes
  int64_t ostride[CDR_MAX_RANK];// output strides in bytes
};

// IDX is the type the unit index is decomposed in: 32-bit when the unit count allows it (a 64-bit
// division costs several times a 32-bit one, and a rank-4 view needs four per 16 bytes moved).
template <int UNIT, typename IDX>
__global__ void __launch_bounds__(256) strided_copy_kernel(const __grid_constant__ CopyArgs a) {
  const IDX step = static_cast<IDX>(gridDim.x) * 256;
  const IDX n_units = static_cast<IDX>(a.n_units);
  for (IDX u = static_cast<IDX>(blockIdx.x) * 256 + threadIdx.x; u < n_units; u += step) {
    IDX rest = u;
    int64_t off = 0, ooff = 0;
#pragma unroll 1
    for (int d = a.rank - 1; d >= 0; --d) {
      const IDX extent = static_cast<IDX>(a.shape[d]);
      const IDX q = rest / extent;
      const int64_t r = static_cast<int64_t>(rest - q * extent);
      off += r * a.stride[d];
      ooff += r * a.ostride[d];
      rest = q;
    }
    if (UNIT == 16) {
      st_stream16(a.out + ooff, ld_stream16(a.in + off));
    } else if (UNIT == 8) {
      *reinterpret_cast<uint64_t*>(a.out + ooff) = *reinterpret_cast<const uint64_t*>(a.in + off);
    } else if (UNIT == 4) {
      *reinterpret_cast<uint32_t*>(a.out + ooff) = *reinterpret_cast<const uint32_t*>(a.in + off);
    } else if (UNIT == 2) {
      *reinterpret_cast<uint16_t*>(a.out + ooff) = *reinterpret_cast<const uint16_t*>(a.in + off);
    } else {
      a.out[ooff] = a.in[off];
    }
  }
}

}  // namespace

int launch_strided_copy(const cdr_tensor* ins, int n_in, const cdr_tensor* outs, int n_out, cudaStream_t stream) {
  if (n_in != 1 || n_out != 1 || !ins || !outs) { set_error("copy: expects one input and one output"); return CDR_ERR_BAD_ARG; }
  const cdr_tensor& x = ins[0];
  const cdr_tensor& out = outs[0];
  if (x.rank != out.rank || x.dtype != out.dtype) { set_error("copy: input and output differ in rank or dtype"); return CDR_ERR_BAD_ARG; }
  for (int d = 0; d < x.rank; ++d)
    if (x.shape[d] != out.shape[d]) { set_error("copy: input and output differ in shape"); return CDR_ERR_BAD_ARG; }
  const int64_t n = numel(out);
  if (n == 0) return CDR_OK;
  if (!x.data || !out.data) { set_error("copy: null pointer"); return CDR_ERR_BAD_ARG; }
  const int esz = dtype_size(x.dtype);
  if (esz <= 0) { set_error("copy: dtype %d unsupported", x.dtype); return CDR_ERR_UNSUPPORTED; }
  for (int d = 0; d < x.rank; ++d) {
    if (x.stride[d] < 0 || out.stride[d] < 0) { set_error("copy: negative strides are not supported"); return CDR_ERR_UNSUPPORTED; }
    if (out.stride[d] == 0 && out.shape[d] > 1) { set_error("copy: the output view overlaps itself (stride 0)"); return CDR_ERR_BAD_ARG; }
  }

  CopyArgs a{};
  a.in = static_cast<const unsigned char*>(x.data);
  a.out = static_cast<unsigned char*>(out.data);
  a.rank = x.rank;
  for (int d = 0; d < x.rank; ++d) {
    a.shape[d] = x.shape[d];
    a.stride[d] = x.stride[d] * esz;
    a.ostride[d] = out.stride[d] * esz;
  }
  if (a.rank == 0) { a.rank = 1; a.shape[0] = 1; a.stride[0] = 0; a.ostride[0] = 0; }
  // vector path: innermost dimension contiguous on both sides, a whole number of 16-byte vectors,
  // every other stride and both base pointers 16-byte aligned
  const int last = a.rank - 1;
  const int per_vec = 16 / esz;
  bool vec = x.rank > 0 && x.stride[last] == 1 && out.stride[last] == 1 && x.shape[last] % per_vec == 0 &&
             aligned16(x.data) && aligned16(out.data);
  for (int d = 0; d < last; ++d) vec &= a.shape[d] == 1 || ((a.stride[d] % 16) == 0 && (a.ostride[d] % 16) == 0);
  if (vec) {
    a.unit_bytes = 16;
    a.shape[last] = x.shape[last] / per_vec;
    a.stride[last] = 16;
    a.ostride[last] = 16;
    a.n_units = n / per_vec;
  } else {
    a.unit_bytes = esz;
    a.n_units = n;
  }
  int64_t grid = (a.n_units + 255) / 256;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
  if (grid > cap) grid = cap;
  const unsigned g = static_cast<unsigned>(grid);
  // the grid-stride loop's index may run one stride past n_units before it stops
  const bool narrow = a.n_units + grid * 256 < (int64_t{1} << 32);
#define CDR_COPY_LAUNCH(UNIT)                                                     \
  if (narrow) strided_copy_kernel<UNIT, uint32_t><<<g, 256, 0, stream>>>(a);      \
  else strided_copy_kernel<UNIT, int64_t><<<g, 256, 0, stream>>>(a)
  switch (a.unit_bytes) {
    case 16: CDR_COPY_LAUNCH(16); break;
    case 8: CDR_COPY_LAUNCH(8); break;
    case 4: CDR_COPY_LAUNCH(4); break;
    case 2: CDR_COPY_LAUNCH(2); break;
    default: CDR_COPY_LAUNCH(1); break;
  }
#undef CDR_COPY_LAUNCH
  CDR_CUDA_TRY(cudaGetLastError());
  return CDR_OK;
}

}  // namespace cdr
