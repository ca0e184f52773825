// Host-buffer forms of matmul / dot: upload, multiply, download as one pipelined
// call.  In the reference these are three separate steps, each a full pass:
// the operands are built on the CPU and copied with `memcpy_stod`
// (crates/hodu_core/src/be/device.rs:35-55), the product runs
// (crates/hodu_core/src/be_cuda/storage/ops_matrix.rs:10-93,95-169), and
// `to_cpu_storage` copies the result back (crates/hodu_core/src/be_cuda/storage.rs:165-173).
// Here the operands are cut into slices (whole batches, or row blocks of the lhs
// when there is one matrix) that rotate over a few streams, so the copy engines
// and the tensor cores overlap; the kernels are the same ones the device forms use.
#include <stdlib.h>

#include <mutex>

#include "common.cuh"

namespace hodu_b200 {
namespace {

constexpr int kSlots = 4;
constexpr int kMaxSlices = 64;

// Tuning knobs read once from the environment: HODU_B200_HOST_SLICES (slices per call, default
// 8) and HODU_B200_HOST_LANES (1, the default: one stream per direction -- upload, compute,
// download -- chained by events; 0: each slice's three steps on one of four rotating streams),
// HODU_B200_HOST_PANELS (column panels of a single large rhs, default 4; 1: upload it whole).
// On a PCIe 5 x16 B200 the schedules differ by a few per cent only: the 16x2048^3 bf16 product
// (256 MiB up, 128 MiB down) takes 5.8-6.1 ms under all of them, against 5.2 ms for the two bare
// copies issued together.
int env_int(const char* name, int dflt, int lo, int hi) {
  const char* e = getenv(name);
  if (!e || !*e) return dflt;
  const int v = atoi(e);
  return v < lo ? lo : (v > hi ? hi : v);
}
int host_slices() { static const int v = env_int("HODU_B200_HOST_SLICES", 8, 1, kMaxSlices); return v; }
int host_panels() { static const int v = env_int("HODU_B200_HOST_PANELS", 4, 1, 8); return v; }
bool host_lanes() { static const int v = env_int("HODU_B200_HOST_LANES", 1, 0, 1); return v != 0; }

struct HostPipe {
  bool ready = false;
  cudaStream_t stream[kSlots] = {};
  cudaEvent_t rhs_ready = nullptr;
  cudaEvent_t uploaded[kMaxSlices] = {}, computed[kMaxSlices] = {};
  void* buf[3] = {nullptr, nullptr, nullptr};  // lhs, rhs, out staging (grow-only)
  size_t cap[3] = {0, 0, 0};
  std::mutex mu;  // one host-form call per device at a time: they share the staging
};
HostPipe g_pipe[kMaxDevices];

int ensure(HostPipe* hp, const size_t need[3]) {
  if (!hp->ready) {
    for (int i = 0; i < kSlots; ++i)
      HODU_CUDA_TRY(cudaStreamCreateWithFlags(&hp->stream[i], cudaStreamNonBlocking), HODU_B200_ERR_LAUNCH);
    HODU_CUDA_TRY(cudaEventCreateWithFlags(&hp->rhs_ready, cudaEventDisableTiming), HODU_B200_ERR_LAUNCH);
    for (int i = 0; i < kMaxSlices; ++i) {
      HODU_CUDA_TRY(cudaEventCreateWithFlags(&hp->uploaded[i], cudaEventDisableTiming), HODU_B200_ERR_LAUNCH);
      HODU_CUDA_TRY(cudaEventCreateWithFlags(&hp->computed[i], cudaEventDisableTiming), HODU_B200_ERR_LAUNCH);
    }
    hp->ready = true;
  }
  for (int i = 0; i < 3; ++i) {
    if (need[i] <= hp->cap[i]) continue;
    if (hp->buf[i]) {
      HODU_CUDA_TRY(cudaDeviceSynchronize(), HODU_B200_ERR_LAUNCH);
      HODU_CUDA_TRY(cudaFree(hp->buf[i]), HODU_B200_ERR_MEMORY);
      hp->buf[i] = nullptr;
      hp->cap[i] = 0;
    }
    HODU_CUDA_TRY(cudaMalloc(&hp->buf[i], need[i]), HODU_B200_ERR_MEMORY);
    hp->cap[i] = need[i];
  }
  return 0;
}

// Records `ev` on `from` and makes `to` wait for it: work queued on `to` afterwards starts when
// everything queued on `from` so far is done.
int hand_over(cudaEvent_t ev, cudaStream_t from, cudaStream_t to) {
  HODU_CUDA_TRY(cudaEventRecord(ev, from), HODU_B200_ERR_LAUNCH);
  HODU_CUDA_TRY(cudaStreamWaitEvent(to, ev, 0), HODU_B200_ERR_LAUNCH);
  return 0;
}

bool contiguous_operand(const Problem& pb, const Operand& op, int64_t rows, int64_t cols, int64_t* elems) {
  // Row-major, offset 0, batch dims densely packed or broadcast as a whole.
  if (op.offset != 0) return false;
  if (!((op.stride_c == 1 || cols == 1) && (op.stride_r == cols || rows == 1))) return false;
  int64_t expect = rows * cols;
  bool any = false, all = true;
  for (int d = pb.batch_ndim - 1; d >= 0; --d) {
    if (pb.batch_shape[d] == 1) continue;
    if (op.bstride[d] == 0) { all = false; continue; }
    any = true;
    if (op.bstride[d] != expect) return false;
    expect *= pb.batch_shape[d];
  }
  if (any && !all) return false;  // partly broadcast: not a fresh tensor's layout
  *elems = any ? expect : rows * cols;
  return true;
}

int host_impl(bool is_dot, int device, int in_dtype, int out_dtype, const void* lhs, const void* rhs,
              void* out, const size_t* md, size_t len, float sl, float sr) {
  Problem pb;
  int r = is_dot ? parse_dot(md, len, &pb) : parse_matmul(md, len, &pb);
  if (r) return r;
  r = check_operands(in_dtype, out_dtype, lhs, rhs, out, sl, sr, 0);
  if (r) return r;
  if (pb.M == 0 || pb.N == 0 || pb.batches == 0) return 0;
  if (pb.K == 0) return fail(HODU_B200_ERR_INVALID_INPUT, "host form: K == 0");
  int64_t a_elems = 0, b_elems = 0;
  if (!contiguous_operand(pb, pb.a, pb.M, pb.K, &a_elems) || !contiguous_operand(pb, pb.b, pb.K, pb.N, &b_elems))
    return fail(HODU_B200_ERR_INVALID_INPUT, "host form: operands must be contiguous with offset 0");
  DeviceState* st = device_state(device);
  if (!st) return HODU_B200_ERR_NOT_INITIALISED;
  DeviceGuard guard(device);
  if (!guard.ok) return fail(HODU_B200_ERR_LAUNCH, "cannot select CUDA device %d", device);

  const int isz = dtype_size(in_dtype), osz = dtype_size(out_dtype);
  const int64_t c_elems = pb.batches * pb.M * pb.N;
  HostPipe* hp = &g_pipe[device];
  std::lock_guard<std::mutex> lock(hp->mu);
  const size_t need[3] = {static_cast<size_t>(a_elems) * isz, static_cast<size_t>(b_elems) * isz,
                          static_cast<size_t>(c_elems) * osz};
  r = ensure(hp, need);
  if (r) return r;
  // Whatever way this call ends, nothing it queued may still be running when the lock is dropped
  // and the caller gets its host buffers back: an early error return would otherwise leave copies
  // in flight that read `lhs` / `rhs`, write `out`, or use the staging the next call overwrites.
  struct DrainOnExit {
    HostPipe* hp;
    ~DrainOnExit() { for (int i = 0; i < kSlots; ++i) cudaStreamSynchronize(hp->stream[i]); }
  } drain{hp};

  pb.in_dtype = in_dtype; pb.out_dtype = out_dtype; pb.alpha = sl * sr;
  const bool lanes = host_lanes();
  const bool a_batched = a_elems > pb.M * pb.K, b_batched = b_elems > pb.K * pb.N;
  const uint8_t* hl = static_cast<const uint8_t*>(lhs);
  const uint8_t* hr = static_cast<const uint8_t*>(rhs);
  uint8_t* ho = static_cast<uint8_t*>(out);
  uint8_t* dl = static_cast<uint8_t*>(hp->buf[0]);
  uint8_t* dr = static_cast<uint8_t*>(hp->buf[1]);
  uint8_t* dout = static_cast<uint8_t*>(hp->buf[2]);

  if (pb.batches > 1 && a_batched && b_batched) {
    // Slices of whole batches: both operands of a slice travel with it.
    const int64_t per = (pb.batches + host_slices() - 1) / host_slices();
    int slot = 0, idx = 0;
    for (int64_t b0 = 0; b0 < pb.batches; b0 += per, slot = (slot + 1) % kSlots, ++idx) {
      const int64_t nb = b0 + per <= pb.batches ? per : pb.batches - b0;
      cudaStream_t s = lanes ? hp->stream[0] : hp->stream[slot];
      const size_t ao = static_cast<size_t>(b0) * pb.M * pb.K * isz, bo = static_cast<size_t>(b0) * pb.K * pb.N * isz;
      const size_t co = static_cast<size_t>(b0) * pb.M * pb.N * osz;
      HODU_CUDA_TRY(cudaMemcpyAsync(dl + ao, hl + ao, static_cast<size_t>(nb) * pb.M * pb.K * isz, cudaMemcpyHostToDevice, s), HODU_B200_ERR_MEMORY);
      HODU_CUDA_TRY(cudaMemcpyAsync(dr + bo, hr + bo, static_cast<size_t>(nb) * pb.K * pb.N * isz, cudaMemcpyHostToDevice, s), HODU_B200_ERR_MEMORY);
      Problem q = pb;
      q.batch_ndim = 1; q.batch_shape[0] = nb; q.batches = nb;
      q.a.ptr = dl + ao; q.a.bstride[0] = pb.M * pb.K; q.a.stride_r = pb.K; q.a.stride_c = 1;
      q.b.ptr = dr + bo; q.b.bstride[0] = pb.K * pb.N; q.b.stride_r = pb.N; q.b.stride_c = 1;
      q.out = dout + co;
      if (lanes) { r = hand_over(hp->uploaded[idx], s, hp->stream[1]); if (r) return r; s = hp->stream[1]; }
      r = run_problem(q, st, s);
      if (r) return r;
      if (lanes) { r = hand_over(hp->computed[idx], s, hp->stream[2]); if (r) return r; s = hp->stream[2]; }
      HODU_CUDA_TRY(cudaMemcpyAsync(ho + co, dout + co, static_cast<size_t>(nb) * pb.M * pb.N * osz, cudaMemcpyDeviceToHost, s), HODU_B200_ERR_MEMORY);
    }
  } else if ((pb.batches == 1 || (!b_batched && a_batched)) && lanes && host_panels() > 1 &&
             pb.N >= 512 * host_panels() && static_cast<size_t>(b_elems) * isz >= (size_t(8) << 20)) {
    // One large rhs for every row of the (flattened) lhs.  Waiting for the whole rhs before the
    // first product would delay the first download by its upload time, so the rhs travels in
    // column panels as well: block (i, j) of the output needs row block i of the lhs and panel j
    // of the rhs only.  Panels and output blocks are pitched (2-D) copies; the kernels write
    // their block straight into the full-size output.
    const int64_t rows = a_batched ? pb.batches * pb.M : pb.M;
    const int panels = host_panels();
    int64_t nbw = (pb.N + panels - 1) / panels;
    nbw = (nbw + 255) / 256 * 256;
    int row_blocks = kMaxSlices / panels < host_slices() ? kMaxSlices / panels : host_slices();
    if (row_blocks > 4) row_blocks = 4;
    int64_t per = (rows + row_blocks - 1) / row_blocks;
    per = (per + 127) / 128 * 128;
    cudaStream_t up = hp->stream[0], comp = hp->stream[1], down = hp->stream[2];
    const int n_panels = static_cast<int>((pb.N + nbw - 1) / nbw), n_rows = static_cast<int>((rows + per - 1) / per);
    if (n_panels * n_rows > kMaxSlices) return fail(HODU_B200_ERR_INVALID_INPUT, "host form: too many blocks");
    auto upload_panel = [&](int j) -> int {
      const int64_t c0 = j * nbw, nc = c0 + nbw <= pb.N ? nbw : pb.N - c0;
      HODU_CUDA_TRY(cudaMemcpy2DAsync(dr + c0 * isz, pb.N * isz, hr + c0 * isz, pb.N * isz, nc * isz, pb.K,
                                      cudaMemcpyHostToDevice, up), HODU_B200_ERR_MEMORY);
      return 0;
    };
    auto upload_rows = [&](int i) -> int {
      const int64_t r0 = i * per, nr = r0 + per <= rows ? per : rows - r0;
      const size_t ao = static_cast<size_t>(r0) * pb.K * isz;
      HODU_CUDA_TRY(cudaMemcpyAsync(dl + ao, hl + ao, static_cast<size_t>(nr) * pb.K * isz, cudaMemcpyHostToDevice, up), HODU_B200_ERR_MEMORY);
      return 0;
    };
    int idx = 0;
    auto block = [&](int i, int j) -> int {   // product and download of output block (i, j)
      const int64_t r0 = i * per, nr = r0 + per <= rows ? per : rows - r0;
      const int64_t c0 = j * nbw, nc = c0 + nbw <= pb.N ? nbw : pb.N - c0;
      const size_t co = (static_cast<size_t>(r0) * pb.N + c0) * osz;
      Problem q = pb;
      q.batch_ndim = 0; q.batches = 1; q.M = nr; q.N = nc;
      q.a.ptr = dl + static_cast<size_t>(r0) * pb.K * isz; q.a.stride_r = pb.K; q.a.stride_c = 1;
      q.b.ptr = dr + c0 * isz; q.b.stride_r = pb.N; q.b.stride_c = 1;
      q.out = dout + co; q.ldc = pb.N;
      int rr = hand_over(hp->uploaded[idx], up, comp);
      if (rr) return rr;
      rr = run_problem(q, st, comp);
      if (rr) return rr;
      rr = hand_over(hp->computed[idx], comp, down);
      if (rr) return rr;
      ++idx;
      HODU_CUDA_TRY(cudaMemcpy2DAsync(ho + co, pb.N * osz, dout + co, pb.N * osz, nc * osz, nr,
                                      cudaMemcpyDeviceToHost, down), HODU_B200_ERR_MEMORY);
      return 0;
    };
    // Uploads alternate between a panel and a row block, so the set of blocks that can be
    // computed grows as a square (1, 2, 4, 6, 9, ..) and the download never waits long.
    int have_rows = 0, have_panels = 0;
    while (have_rows < n_rows || have_panels < n_panels) {
      const bool take_panel = have_panels < n_panels && (have_panels <= have_rows || have_rows == n_rows);
      if (take_panel) {
        if ((r = upload_panel(have_panels))) return r;
        for (int i = 0; i < have_rows; ++i)
          if ((r = block(i, have_panels))) return r;
        ++have_panels;
      } else {
        if ((r = upload_rows(have_rows))) return r;
        for (int j = 0; j < have_panels; ++j)
          if ((r = block(have_rows, j))) return r;
        ++have_rows;
      }
    }
  } else if (pb.batches == 1 || (!b_batched && a_batched)) {
    // One rhs for every row of the (flattened) lhs: upload it once, then stream
    // row blocks of the lhs through the slots.
    const int64_t rows = a_batched ? pb.batches * pb.M : pb.M;
    HODU_CUDA_TRY(cudaMemcpyAsync(dr, hr, static_cast<size_t>(b_elems) * isz, cudaMemcpyHostToDevice, hp->stream[0]), HODU_B200_ERR_MEMORY);
    HODU_CUDA_TRY(cudaEventRecord(hp->rhs_ready, hp->stream[0]), HODU_B200_ERR_LAUNCH);
    int64_t per = (rows + host_slices() - 1) / host_slices();
    per = (per + 127) / 128 * 128;
    int slot = 0, idx = 0;
    for (int64_t r0 = 0; r0 < rows; r0 += per, slot = (slot + 1) % kSlots, ++idx) {
      const int64_t nr = r0 + per <= rows ? per : rows - r0;
      cudaStream_t s = lanes ? hp->stream[0] : hp->stream[slot];
      const size_t ao = static_cast<size_t>(r0) * pb.K * isz, co = static_cast<size_t>(r0) * pb.N * osz;
      HODU_CUDA_TRY(cudaMemcpyAsync(dl + ao, hl + ao, static_cast<size_t>(nr) * pb.K * isz, cudaMemcpyHostToDevice, s), HODU_B200_ERR_MEMORY);
      if (!lanes) HODU_CUDA_TRY(cudaStreamWaitEvent(s, hp->rhs_ready, 0), HODU_B200_ERR_LAUNCH);
      Problem q = pb;
      q.batch_ndim = 0; q.batches = 1; q.M = nr;
      q.a.ptr = dl + ao; q.a.stride_r = pb.K; q.a.stride_c = 1;
      q.b.ptr = dr; q.b.stride_r = pb.N; q.b.stride_c = 1;
      q.out = dout + co;
      if (lanes) { r = hand_over(hp->uploaded[idx], s, hp->stream[1]); if (r) return r; s = hp->stream[1]; }
      r = run_problem(q, st, s);
      if (r) return r;
      if (lanes) { r = hand_over(hp->computed[idx], s, hp->stream[2]); if (r) return r; s = hp->stream[2]; }
      HODU_CUDA_TRY(cudaMemcpyAsync(ho + co, dout + co, static_cast<size_t>(nr) * pb.N * osz, cudaMemcpyDeviceToHost, s), HODU_B200_ERR_MEMORY);
    }
  } else {
    // Broadcast lhs: no slicing, one pass.
    cudaStream_t s = hp->stream[0];
    HODU_CUDA_TRY(cudaMemcpyAsync(dl, hl, static_cast<size_t>(a_elems) * isz, cudaMemcpyHostToDevice, s), HODU_B200_ERR_MEMORY);
    HODU_CUDA_TRY(cudaMemcpyAsync(dr, hr, static_cast<size_t>(b_elems) * isz, cudaMemcpyHostToDevice, s), HODU_B200_ERR_MEMORY);
    Problem q = pb;
    q.a.ptr = dl; q.b.ptr = dr; q.out = dout;
    r = run_problem(q, st, s);
    if (r) return r;
    HODU_CUDA_TRY(cudaMemcpyAsync(ho, dout, static_cast<size_t>(c_elems) * osz, cudaMemcpyDeviceToHost, s), HODU_B200_ERR_MEMORY);
  }
  for (int i = 0; i < kSlots; ++i) HODU_CUDA_TRY(cudaStreamSynchronize(hp->stream[i]), HODU_B200_ERR_LAUNCH);
  return 0;
}

// SwiGLU MLP over host activations: tokens travel in row blocks, the three weight matrices stay
// where they are (device memory).  Block i: upload x_i -> hidden_i = silu(x_i.Wg) * (x_i.Wu) ->
// y_i = hidden_i . Wd -> download y_i, on the same three streams as above, so the upload of block
// i+1 and the download of block i-1 run under the two products of block i.
int mlp_host_impl(int device, int dtype, const void* x_host, const void* w_gate, const void* w_up,
                  const void* w_down, void* y_host, const size_t* md, size_t len, uint32_t flags) {
  if (!md || len != 13) return fail(HODU_B200_ERR_INVALID_INPUT, "swiglu_mlp_host: metadata length %zu, expected 13", len);
  if (dtype != HODU_DTYPE_BF16 && dtype != HODU_DTYPE_F16)
    return fail(HODU_B200_ERR_INVALID_KERNEL, "swiglu_mlp_host: unsupported dtype %s", dtype_name(dtype));
  if (flags != HODU_B200_SWIGLU_ROUND_EACH_OP && flags != HODU_B200_SWIGLU_ROUND_ONCE)
    return fail(HODU_B200_ERR_INVALID_INPUT, "swiglu_mlp_host: unknown flags %u", flags);
  for (int i = 0; i < 4; ++i)
    if (md[i] > (1ull << 32)) return fail(HODU_B200_ERR_INVALID_INPUT, "swiglu_mlp_host: extent out of range");
  for (int i = 4; i < 13; ++i)
    if (md[i] > (1ull << 48)) return fail(HODU_B200_ERR_INVALID_INPUT, "swiglu_mlp_host: stride or offset out of range");
  const int64_t tokens = md[0], d_in = md[1], d_hidden = md[2], d_out = md[3];
  if (tokens == 0 || d_out == 0) return 0;
  if (d_in == 0 || d_hidden == 0) return fail(HODU_B200_ERR_INVALID_INPUT, "swiglu_mlp_host: empty feature dimension");
  if (!x_host || !w_gate || !w_up || !w_down || !y_host) return fail(HODU_B200_ERR_INVALID_INPUT, "null operand pointer");
  DeviceState* st = device_state(device);
  if (!st) return HODU_B200_ERR_NOT_INITIALISED;
  DeviceGuard guard(device);
  if (!guard.ok) return fail(HODU_B200_ERR_LAUNCH, "cannot select CUDA device %d", device);

  const int esz = dtype_size(dtype);
  int64_t per = (tokens + host_slices() - 1) / host_slices();
  per = (per + 511) / 512 * 512;   // whole 512-row tiles per block
  const int n_blocks = static_cast<int>((tokens + per - 1) / per);
  if (n_blocks > kMaxSlices) return fail(HODU_B200_ERR_INVALID_INPUT, "swiglu_mlp_host: too many blocks");
  HostPipe* hp = &g_pipe[device];
  std::lock_guard<std::mutex> lock(hp->mu);
  // staging: all of x, ONE hidden block (the products run in order on one stream), all of y
  const size_t need[3] = {static_cast<size_t>(tokens) * d_in * esz, static_cast<size_t>(per) * d_hidden * esz,
                          static_cast<size_t>(tokens) * d_out * esz};
  int r = ensure(hp, need);
  if (r) return r;
  struct DrainOnExit {
    HostPipe* hp;
    ~DrainOnExit() { for (int i = 0; i < kSlots; ++i) cudaStreamSynchronize(hp->stream[i]); }
  } drain{hp};
  const uint8_t* hx = static_cast<const uint8_t*>(x_host);
  uint8_t* hy = static_cast<uint8_t*>(y_host);
  uint8_t* dx = static_cast<uint8_t*>(hp->buf[0]);
  uint8_t* dh = static_cast<uint8_t*>(hp->buf[1]);
  uint8_t* dy = static_cast<uint8_t*>(hp->buf[2]);
  cudaStream_t up = hp->stream[0], comp = hp->stream[1], down = hp->stream[2];
  for (int i = 0; i < n_blocks; ++i) {
    const int64_t r0 = i * per, nr = r0 + per <= tokens ? per : tokens - r0;
    const size_t xo = static_cast<size_t>(r0) * d_in * esz, yo = static_cast<size_t>(r0) * d_out * esz;
    HODU_CUDA_TRY(cudaMemcpyAsync(dx + xo, hx + xo, static_cast<size_t>(nr) * d_in * esz, cudaMemcpyHostToDevice, up), HODU_B200_ERR_MEMORY);
    if ((r = hand_over(hp->uploaded[i], up, comp))) return r;
    Problem g;
    g.in_dtype = dtype; g.out_dtype = dtype;
    g.M = nr; g.K = d_in; g.N = d_hidden;
    g.a.ptr = dx + xo; g.a.stride_r = d_in; g.a.stride_c = 1;
    g.b.ptr = w_gate; g.b.stride_r = md[4]; g.b.stride_c = md[5]; g.b.offset = md[10];
    g.b2.ptr = w_up; g.b2.stride_r = md[6]; g.b2.stride_c = md[7]; g.b2.offset = md[11];
    g.swiglu = true; g.swiglu_flags = flags;
    g.out = dh;
    if ((r = run_problem(g, st, comp))) return r;
    Problem d;
    d.in_dtype = dtype; d.out_dtype = dtype;
    d.M = nr; d.K = d_hidden; d.N = d_out;
    d.a.ptr = dh; d.a.stride_r = d_hidden; d.a.stride_c = 1;
    d.b.ptr = w_down; d.b.stride_r = md[8]; d.b.stride_c = md[9]; d.b.offset = md[12];
    d.out = dy + yo;
    if ((r = run_problem(d, st, comp))) return r;
    if ((r = hand_over(hp->computed[i], comp, down))) return r;
    HODU_CUDA_TRY(cudaMemcpyAsync(hy + yo, dy + yo, static_cast<size_t>(nr) * d_out * esz, cudaMemcpyDeviceToHost, down), HODU_B200_ERR_MEMORY);
  }
  for (int i = 0; i < kSlots; ++i) HODU_CUDA_TRY(cudaStreamSynchronize(hp->stream[i]), HODU_B200_ERR_LAUNCH);
  return 0;
}

}  // namespace

void release_host_pipeline(int device) {
  HostPipe* hp = &g_pipe[device];
  std::lock_guard<std::mutex> lock(hp->mu);
  for (int i = 0; i < 3; ++i) {
    if (hp->buf[i]) cudaFree(hp->buf[i]);
    hp->buf[i] = nullptr;
    hp->cap[i] = 0;
  }
  if (hp->ready) {
    for (int i = 0; i < kSlots; ++i) cudaStreamDestroy(hp->stream[i]);
    cudaEventDestroy(hp->rhs_ready);
    for (int i = 0; i < kMaxSlices; ++i) { cudaEventDestroy(hp->uploaded[i]); cudaEventDestroy(hp->computed[i]); }
    hp->ready = false;
  }
}

}  // namespace hodu_b200

using namespace hodu_b200;

extern "C" {
int hodu_b200_matmul_host(int device, uint8_t in_dtype, uint8_t out_dtype, const void* lhs, const void* rhs,
                          void* out, const size_t* md, size_t len, float sl, float sr) {
  return host_impl(false, device, in_dtype, out_dtype, lhs, rhs, out, md, len, sl, sr);
}
int hodu_b200_dot_host(int device, uint8_t in_dtype, uint8_t out_dtype, const void* lhs, const void* rhs,
                       void* out, const size_t* md, size_t len, float sl, float sr) {
  return host_impl(true, device, in_dtype, out_dtype, lhs, rhs, out, md, len, sl, sr);
}
int hodu_b200_swiglu_mlp_host(int device, uint8_t dtype, const void* x_host, const void* w_gate, const void* w_up,
                              const void* w_down, void* y_host, const size_t* md, size_t len, uint32_t flags) {
  return mlp_host_impl(device, dtype, x_host, w_gate, w_up, w_down, y_host, md, len, flags);
}
}
