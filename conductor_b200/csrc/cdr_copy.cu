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
// 16-byte vector with streaming accesses.  When the view's unit-stride dimension is NOT its
// innermost one (a transpose: x.t(), permute(0, 2, 1), [B, S, H, D] -> [B, H, D, S]) a tile of
// (that dimension) x (innermost dimension) goes through shared memory, so that both the reads
// and the writes run along memory; every other dimension is a batch index.  Anything else is
// gathered element by element (reads uncoalesced when no dimension of the view has stride 1).
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

// ---- transpose through shared memory --------------------------------------------------------
struct TransposeArgs {
  const unsigned char* in;
  unsigned char* out;
  int32_t rank, pdim;            // pdim: the view dimension whose input stride is one element
  int64_t shape[CDR_MAX_RANK];
  int64_t stride[CDR_MAX_RANK];  // input strides in bytes
  int64_t ostride[CDR_MAX_RANK]; // output strides in bytes
  int64_t tiles_p, tiles_l;      // tiles along pdim and along the innermost dimension
};

// T: an unsigned integer of the element's size.  TILE x TILE elements per CTA of 256 threads; the
// shared tile is padded by one 32-bit word per row, so column reads hit distinct banks.
template <typename T, int TILE>
__global__ void __launch_bounds__(256) transpose_tile_kernel(const __grid_constant__ TransposeArgs a) {
  constexpr int PAD = sizeof(T) >= 4 ? 1 : 4 / sizeof(T);
  constexpr int ROWS = 256 / TILE;          // tile rows handled per pass
  __shared__ T tile[TILE][TILE + PAD];
  const int last = a.rank - 1;
  int64_t b = blockIdx.x;
  const int64_t tl = b % a.tiles_l; b /= a.tiles_l;
  const int64_t tp = b % a.tiles_p; b /= a.tiles_p;
  int64_t in_base = 0, out_base = 0;       // the batch dimensions: every one but pdim and the innermost
#pragma unroll 1
  for (int d = last - 1; d >= 0; --d) {
    if (d == a.pdim) continue;
    const int64_t q = b / a.shape[d], r = b - q * a.shape[d];
    in_base += r * a.stride[d];
    out_base += r * a.ostride[d];
    b = q;
  }
  const int64_t p0 = tp * TILE, l0 = tl * TILE;
  const int tx = threadIdx.x % TILE, ty = threadIdx.x / TILE;
  // read: consecutive threads along pdim (unit stride in memory), rows of the tile along the innermost dimension
#pragma unroll
  for (int y = ty; y < TILE; y += ROWS) {
    const int64_t pi = p0 + tx, li = l0 + y;
    if (pi < a.shape[a.pdim] && li < a.shape[last])
      tile[y][tx] = *reinterpret_cast<const T*>(a.in + in_base + pi * a.stride[a.pdim] + li * a.stride[last]);
  }
  __syncthreads();
  // write: consecutive threads along the innermost dimension (unit stride in the output)
#pragma unroll
  for (int y = ty; y < TILE; y += ROWS) {
    const int64_t pi = p0 + y, li = l0 + tx;
    if (pi < a.shape[a.pdim] && li < a.shape[last])
      *reinterpret_cast<T*>(a.out + out_base + pi * a.ostride[a.pdim] + li * a.ostride[last]) = tile[tx][y];
  }
}

// Vector form of the tile transpose: every thread moves 16 bytes on both sides (V elements along the
// input's unit-stride dimension on the way in, V elements along the output's on the way out), so a
// warp request covers whole 128-byte lines for 2-byte types too.  Needs every extent, stride and
// base involved to be a multiple of 16 bytes; the scalar form above takes the rest.
template <typename T>
__global__ void __launch_bounds__(256) transpose_tile_vec_kernel(const __grid_constant__ TransposeArgs a) {
  constexpr int V = 16 / sizeof(T);
  constexpr int TILE = 16 * V;
  constexpr int PAD = sizeof(T) >= 4 ? 1 : 4 / sizeof(T);
  __shared__ T tile[TILE][TILE + PAD];
  const int last = a.rank - 1;
  int64_t b = blockIdx.x;
  const int64_t tl = b % a.tiles_l; b /= a.tiles_l;
  const int64_t tp = b % a.tiles_p; b /= a.tiles_p;
  int64_t in_base = 0, out_base = 0;
#pragma unroll 1
  for (int d = last - 1; d >= 0; --d) {
    if (d == a.pdim) continue;
    const int64_t q = b / a.shape[d], r = b - q * a.shape[d];
    in_base += r * a.stride[d];
    out_base += r * a.ostride[d];
    b = q;
  }
  const int64_t p0 = tp * TILE, l0 = tl * TILE;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
#pragma unroll 4
  for (int y = ty; y < TILE; y += 16) {
    const int64_t pi = p0 + tx * V, li = l0 + y;
    if (pi < a.shape[a.pdim] && li < a.shape[last]) {
      const uint4 q = ld_stream16(a.in + in_base + pi * a.stride[a.pdim] + li * a.stride[last]);
      const T* e = reinterpret_cast<const T*>(&q);
#pragma unroll
      for (int i = 0; i < V; ++i) tile[y][tx * V + i] = e[i];
    }
  }
  __syncthreads();
#pragma unroll 4
  for (int y = ty; y < TILE; y += 16) {
    const int64_t pi = p0 + y, li = l0 + tx * V;
    if (pi < a.shape[a.pdim] && li < a.shape[last]) {
      uint4 q;
      T* e = reinterpret_cast<T*>(&q);
#pragma unroll
      for (int i = 0; i < V; ++i) e[i] = tile[tx * V + i][y];
      st_stream16(a.out + out_base + pi * a.ostride[a.pdim] + li * a.ostride[last], q);
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
  if (!vec && x.rank >= 2 && out.stride[last] == 1 && x.stride[last] != 1 && x.shape[last] > 1) {
    // a transpose: some other dimension of the view runs along memory in the input
    int pdim = -1;
    for (int d = last - 1; d >= 0; --d)
      if (x.stride[d] == 1 && x.shape[d] > 1) { pdim = d; break; }
    if (pdim >= 0) {
      TransposeArgs t{};
      t.in = a.in; t.out = a.out; t.rank = a.rank; t.pdim = pdim;
      for (int d = 0; d < a.rank; ++d) { t.shape[d] = a.shape[d]; t.stride[d] = a.stride[d]; t.ostride[d] = a.ostride[d]; }
      // 16-byte accesses on both sides when every extent, stride and base allows it
      bool tvec = (esz == 2 || esz == 4 || esz == 8) && aligned16(x.data) && aligned16(out.data) &&
                  x.shape[pdim] % per_vec == 0 && x.shape[last] % per_vec == 0;
      for (int d = 0; d < a.rank && tvec; ++d) {
        if (d != pdim && a.shape[d] > 1) tvec &= (a.stride[d] % 16) == 0;
        if (d != last && a.shape[d] > 1) tvec &= (a.ostride[d] % 16) == 0;
      }
      const int tile = tvec ? 16 * per_vec : 64;   // scalar form: 64 x 64 elements per CTA
      t.tiles_p = (x.shape[pdim] + tile - 1) / tile;
      t.tiles_l = (x.shape[last] + tile - 1) / tile;
      int64_t batch = 1;
      for (int d = 0; d < last; ++d)
        if (d != pdim) batch *= x.shape[d];
      const int64_t blocks = batch * t.tiles_p * t.tiles_l;
      if (blocks > 0 && blocks < (int64_t{1} << 31)) {
        const unsigned g = static_cast<unsigned>(blocks);
        if (tvec) {
          if (esz == 2) transpose_tile_vec_kernel<uint16_t><<<g, 256, 0, stream>>>(t);
          else if (esz == 4) transpose_tile_vec_kernel<uint32_t><<<g, 256, 0, stream>>>(t);
          else transpose_tile_vec_kernel<uint64_t><<<g, 256, 0, stream>>>(t);
          CDR_CUDA_TRY(cudaGetLastError());
          return CDR_OK;
        }
        switch (esz) {
          case 1: transpose_tile_kernel<uint8_t, 64><<<g, 256, 0, stream>>>(t); break;
          case 2: transpose_tile_kernel<uint16_t, 64><<<g, 256, 0, stream>>>(t); break;
          case 4: transpose_tile_kernel<uint32_t, 64><<<g, 256, 0, stream>>>(t); break;
          default: transpose_tile_kernel<uint64_t, 64><<<g, 256, 0, stream>>>(t); break;
        }
        CDR_CUDA_TRY(cudaGetLastError());
        return CDR_OK;
      }
    }
  }
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
