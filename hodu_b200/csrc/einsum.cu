// Two-operand einsum contractions mapped onto the GEMM.
//
// The reference evaluates every einsum with one thread per output element that walks all
// contraction indices (crates/hodu_cuda_kernels/kernels/ops_einsum.cu:76-175; f32 running
// sum, one conversion at the end).  When every index of a two-operand equation is a batch,
// M, N or K index the same sum is a (batched) matrix product over strided views, which is
// what this file recognises: it reads the reference's einsum wire format
// (crates/hodu_core/src/op_metadatas.rs:1502-1567) and fills a `Problem` for `run_problem`.
// Nothing is copied; forms that are not a matrix product are refused with "invalid kernel".
#include <cstdio>

#include "common.cuh"

namespace hodu_b200 {
namespace {

constexpr int kMaxIdx = 16;
constexpr int kMaxDims = 16;

struct EinsumInput {
  size_t ndim = 0;
  size_t shape[kMaxDims];
  size_t stride[kMaxDims];
  size_t offset = 0;
  size_t index_of_dim[kMaxDims];
  int dim_of_index[kMaxIdx];  // -1: index absent from this operand
};

enum Kind { kBatch, kM, kN, kK };

// Merges the dims `ids` (outermost first) of one operand into a single stride.  Extent-1
// dims are skipped.  Returns false if the dims do not lie in memory as one strided run.
bool merge_stride(const EinsumInput& in, const int* ids, int n, const size_t* sizes, int64_t* stride) {
  int64_t inner_stride = 0, inner_extent = 0;
  bool have = false;
  for (int i = n - 1; i >= 0; --i) {
    const size_t sz = sizes[ids[i]];
    if (sz == 1) continue;
    const int64_t s = static_cast<int64_t>(in.stride[in.dim_of_index[ids[i]]]);
    if (!have) {
      *stride = s;
      inner_stride = s;
      inner_extent = static_cast<int64_t>(sz);
      have = true;
    } else {
      if (static_cast<__int128>(s) != static_cast<__int128>(inner_stride) * inner_extent) return false;
      inner_extent *= static_cast<int64_t>(sz);
    }
  }
  if (!have) *stride = 0;  // extent 1 (or no index of this kind): the stride is never used
  return true;
}

}  // namespace

int parse_einsum(const size_t* md, size_t len, size_t num_inputs, Problem* pb, bool* swapped) {
  if (!md || len < 5) return fail(HODU_B200_ERR_INVALID_INPUT, "einsum: metadata too short (%zu)", len);
  const size_t num_out = md[0], n_in = md[1], n_idx = md[2], n_con = md[3], out_ndim = md[4];
  if (n_in != num_inputs)
    return fail(HODU_B200_ERR_INVALID_INPUT, "einsum: metadata names %zu inputs, %zu given", n_in, num_inputs);
  if (n_in != 2)
    return fail(HODU_B200_ERR_INVALID_KERNEL, "einsum: %zu operands; only two-operand contractions run on the GEMM", n_in);
  if (n_idx == 0 || n_idx > kMaxIdx || n_con > n_idx || out_ndim > kMaxDims)
    return fail(HODU_B200_ERR_INVALID_INPUT, "einsum: bad counts (indices %zu, contracted %zu, output dims %zu)", n_idx, n_con, out_ndim);
  size_t pos = 5;
  if (len < pos + out_ndim) return fail(HODU_B200_ERR_INVALID_INPUT, "einsum: metadata truncated (output shape)");
  const size_t* out_shape = md + pos;
  pos += out_ndim;
  EinsumInput in[2];
  for (int i = 0; i < 2; ++i) {
    if (len < pos + 1) return fail(HODU_B200_ERR_INVALID_INPUT, "einsum: metadata truncated (input %d)", i);
    const size_t nd = md[pos++];
    if (nd > kMaxDims) return fail(HODU_B200_ERR_INVALID_INPUT, "einsum: input %d has %zu dims", i, nd);
    if (len < pos + 3 * nd + 1) return fail(HODU_B200_ERR_INVALID_INPUT, "einsum: metadata truncated (input %d)", i);
    in[i].ndim = nd;
    for (size_t d = 0; d < nd; ++d) in[i].shape[d] = md[pos++];
    for (size_t d = 0; d < nd; ++d) in[i].stride[d] = md[pos++];
    in[i].offset = md[pos++];
    for (size_t x = 0; x < n_idx; ++x) in[i].dim_of_index[x] = -1;
    for (size_t d = 0; d < nd; ++d) {
      const size_t id = md[pos++];
      if (id >= n_idx) return fail(HODU_B200_ERR_INVALID_INPUT, "einsum: index id %zu out of range", id);
      if (in[i].dim_of_index[id] >= 0)
        return fail(HODU_B200_ERR_INVALID_KERNEL, "einsum: an index repeated within one operand (diagonal) is not a matrix product");
      in[i].index_of_dim[d] = id;
      in[i].dim_of_index[id] = static_cast<int>(d);
    }
  }
  if (len != pos + n_con + n_idx + out_ndim)
    return fail(HODU_B200_ERR_INVALID_INPUT, "einsum: metadata length %zu, expected %zu", len, pos + n_con + n_idx + out_ndim);
  pos += n_con;  // the contracted ids follow from the output ids below
  const size_t* sizes = md + pos;
  pos += n_idx;
  const size_t* out_ids = md + pos;

  {  // index sizes a real tensor can have: each up to 2^32, all together up to 2^48 elements
    unsigned __int128 total = 1;
    for (size_t x = 0; x < n_idx; ++x) {
      if (sizes[x] > (1ull << 32)) return fail(HODU_B200_ERR_INVALID_INPUT, "einsum: index size %zu out of range", sizes[x]);
      if (sizes[x] > 0) total *= sizes[x];
      if (total > (1ull << 48)) return fail(HODU_B200_ERR_INVALID_INPUT, "einsum: index sizes multiply to more than 2^48");
    }
    for (int i = 0; i < 2; ++i) {
      if (in[i].offset > (1ull << 48)) return fail(HODU_B200_ERR_INVALID_INPUT, "einsum: offset out of range");
      for (size_t dd = 0; dd < in[i].ndim; ++dd)
        if (in[i].stride[dd] > (1ull << 48)) return fail(HODU_B200_ERR_INVALID_INPUT, "einsum: stride out of range");
    }
  }
  int out_dim_of_index[kMaxIdx];
  for (size_t x = 0; x < n_idx; ++x) out_dim_of_index[x] = -1;
  size_t expect_out = 1;
  for (size_t d = 0; d < out_ndim; ++d) {
    const size_t id = out_ids[d];
    if (id >= n_idx) return fail(HODU_B200_ERR_INVALID_INPUT, "einsum: output index id %zu out of range", id);
    if (out_dim_of_index[id] >= 0)
      return fail(HODU_B200_ERR_INVALID_KERNEL, "einsum: an index repeated in the output is not a matrix product");
    if (out_shape[d] != sizes[id]) return fail(HODU_B200_ERR_INVALID_INPUT, "einsum: output dim %zu has extent %zu, index has %zu", d, out_shape[d], sizes[id]);
    out_dim_of_index[id] = static_cast<int>(d);
    expect_out *= out_shape[d];
  }
  // The reference writes max(size, 1) here (a scalar output has one element).
  if (num_out != expect_out && num_out != (expect_out > 0 ? expect_out : 1))
    return fail(HODU_B200_ERR_INVALID_INPUT, "einsum: num_output_els %zu disagrees with the output shape", num_out);
  for (int i = 0; i < 2; ++i)
    for (size_t d = 0; d < in[i].ndim; ++d)
      if (in[i].shape[d] != sizes[in[i].index_of_dim[d]])
        return fail(HODU_B200_ERR_INVALID_INPUT, "einsum: input %d dim %zu has extent %zu, index has %zu", i, d, in[i].shape[d], sizes[in[i].index_of_dim[d]]);

  // Kind of every index.
  Kind kind[kMaxIdx];
  for (size_t x = 0; x < n_idx; ++x) {
    const bool a = in[0].dim_of_index[x] >= 0, b = in[1].dim_of_index[x] >= 0, o = out_dim_of_index[x] >= 0;
    if (a && b && o) kind[x] = kBatch;
    else if (a && !b && o) kind[x] = kM;
    else if (!a && b && o) kind[x] = kN;
    else if (a && b && !o) kind[x] = kK;
    else
      return fail(HODU_B200_ERR_INVALID_KERNEL, "einsum: index %zu is summed over a single operand (or unused); not a matrix product", x);
  }
  // Output order: batch.., then all of one operand's free indices, then the other's.
  int batch_ids[kMaxIdx], first_ids[kMaxIdx], second_ids[kMaxIdx];
  int nb = 0, n1 = 0, n2 = 0;
  Kind first_kind = kM;
  size_t d = 0;
  for (; d < out_ndim && kind[out_ids[d]] == kBatch; ++d) batch_ids[nb++] = static_cast<int>(out_ids[d]);
  if (d < out_ndim) first_kind = kind[out_ids[d]];
  for (; d < out_ndim && kind[out_ids[d]] == first_kind; ++d) first_ids[n1++] = static_cast<int>(out_ids[d]);
  const Kind second_kind = first_kind == kM ? kN : kM;
  for (; d < out_ndim && kind[out_ids[d]] == second_kind; ++d) second_ids[n2++] = static_cast<int>(out_ids[d]);
  if (d != out_ndim)
    return fail(HODU_B200_ERR_INVALID_KERNEL, "einsum: output order interleaves batch / row / column indices; not a contiguous matrix product");
  // lhs = the operand whose free indices come first in the output.
  const bool swap = (n1 > 0 && first_kind == kN);
  *swapped = swap;
  const EinsumInput& A = in[swap ? 1 : 0];
  const EinsumInput& B = in[swap ? 0 : 1];
  // Contracted indices, in the order the lhs holds them (outermost first).
  int k_ids[kMaxIdx];
  int nk = 0;
  for (size_t dd = 0; dd < A.ndim; ++dd)
    if (kind[A.index_of_dim[dd]] == kK) k_ids[nk++] = static_cast<int>(A.index_of_dim[dd]);

  int64_t a_sr = 0, a_sc = 0, b_sr = 0, b_sc = 0;
  if (!merge_stride(A, first_ids, n1, sizes, &a_sr) || !merge_stride(B, second_ids, n2, sizes, &b_sc))
    return fail(HODU_B200_ERR_INVALID_KERNEL, "einsum: the row (or column) indices of an operand do not merge into one stride");
  bool k_ok = merge_stride(A, k_ids, nk, sizes, &a_sc) && merge_stride(B, k_ids, nk, sizes, &b_sr);
  if (!k_ok) {
    // Try the order of the rhs instead.
    nk = 0;
    for (size_t dd = 0; dd < B.ndim; ++dd)
      if (kind[B.index_of_dim[dd]] == kK) k_ids[nk++] = static_cast<int>(B.index_of_dim[dd]);
    k_ok = merge_stride(A, k_ids, nk, sizes, &a_sc) && merge_stride(B, k_ids, nk, sizes, &b_sr);
  }
  if (!k_ok)
    return fail(HODU_B200_ERR_INVALID_KERNEL, "einsum: the contracted indices do not merge into one stride in both operands");

  auto extent = [&](const int* ids, int n) { int64_t e = 1; for (int i = 0; i < n; ++i) e *= static_cast<int64_t>(sizes[ids[i]]); return e; };
  pb->M = extent(first_ids, n1);
  pb->N = extent(second_ids, n2);
  pb->K = extent(k_ids, nk);
  pb->batch_ndim = nb;
  pb->batches = 1;
  for (int i = 0; i < nb; ++i) {
    const int id = batch_ids[i];
    pb->batch_shape[i] = static_cast<int64_t>(sizes[id]);
    pb->batches *= pb->batch_shape[i];
    pb->a.bstride[i] = sizes[id] == 1 ? 0 : static_cast<int64_t>(A.stride[A.dim_of_index[id]]);
    pb->b.bstride[i] = sizes[id] == 1 ? 0 : static_cast<int64_t>(B.stride[B.dim_of_index[id]]);
  }
  // A stride that is never used (extent 1) is given the value a dense matrix would have, so that
  // the layout classification sees an ordinary operand.
  if (pb->K == 1) { a_sc = 1; b_sr = pb->N > 1 && b_sc == 1 ? pb->N : 1; }
  if (pb->M == 1) a_sr = a_sc == 1 ? pb->K : 1;
  if (pb->N == 1) b_sc = b_sr == 1 ? pb->K : 1;
  if (pb->K == 1 && a_sr == 1 && pb->M > 1) a_sc = pb->M;  // column vector: M-contiguous view
  pb->a.stride_r = a_sr; pb->a.stride_c = a_sc;
  pb->b.stride_r = b_sr; pb->b.stride_c = b_sc;
  pb->a.offset = static_cast<int64_t>(A.offset);
  pb->b.offset = static_cast<int64_t>(B.offset);
  return check_extents(*pb);
}

}  // namespace hodu_b200
