"""The host-side mirror of Tensor::matmul / dot / to_dtype / Linear and the host-buffer
entry points, against the oracle."""
import numpy as np
import pytest
import torch

from gpu_util import DEV, from_dev, to_dev
from hodu_b200 import DType, Layout, _lib
from hodu_b200 import kernels as K
from hodu_b200.nn import Linear
from hodu_b200.op_metadatas import dot_metadata, matmul_metadata
from hodu_b200.tensor import HoduError, Tensor
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def bf16_tensor(x):
    return Tensor.from_torch(torch.from_numpy(x).to(DEV).to(torch.bfloat16))


def as_f32(t: Tensor):
    return t.to_torch().float().cpu().numpy()


def ref_matmul(a, b):
    af = O.widen(O.f32_to_bf16(a), O.BF16)
    bf = O.widen(O.f32_to_bf16(b), O.BF16)
    return O.widen(O.narrow(np.matmul(af, bf).astype(np.float32), O.BF16), O.BF16)


def test_rank_dispatch_follows_the_reference():
    rng = np.random.default_rng(0)
    a2, b2 = rng.standard_normal((64, 128)).astype(np.float32), rng.standard_normal((128, 72)).astype(np.float32)
    v = rng.standard_normal(128).astype(np.float32)
    A, B, V = bf16_tensor(a2), bf16_tensor(b2), bf16_tensor(v)
    assert A.matmul(B).shape == (64, 72)
    assert O.rel_err(as_f32(A.matmul(B)), ref_matmul(a2, b2)) <= 1e-2
    assert A.matmul(V).shape == (64,)                       # 2-D x 1-D: reshape, dot, squeeze
    assert O.rel_err(as_f32(A.matmul(V)), ref_matmul(a2, v[:, None])[:, 0]) <= 1e-2
    assert V.matmul(B).shape == (72,)                       # 1-D x 2-D
    assert O.rel_err(as_f32(V.matmul(B)), ref_matmul(v[None, :], b2)[0]) <= 1e-2
    a4 = rng.standard_normal((2, 1, 40, 128)).astype(np.float32)
    b3 = rng.standard_normal((3, 128, 48)).astype(np.float32)
    r = bf16_tensor(a4).matmul(bf16_tensor(b3))             # ND with broadcasting
    assert r.shape == (2, 3, 40, 48)
    assert O.rel_err(as_f32(r), ref_matmul(a4, b3)) <= 1e-2
    with pytest.raises(HoduError):
        A.matmul(A)                                         # 128 != 64
    with pytest.raises(HoduError):
        A.matmul(Tensor.from_torch(torch.zeros(128, 8, device=DEV)))  # dtype mismatch
    with pytest.raises(HoduError):
        bf16_tensor(a4).matmul(bf16_tensor(rng.standard_normal((5, 4, 128, 8)).astype(np.float32)))  # 2 vs 5


def test_linear_forward_uses_the_transposed_view():
    rng = np.random.default_rng(1)
    x = rng.standard_normal((256, 192)).astype(np.float32)
    w = rng.standard_normal((320, 192)).astype(np.float32)   # [out, in]
    y = Linear(bf16_tensor(w)).forward(bf16_tensor(x))
    assert y.shape == (256, 320) and K.last_path() == _lib.PATH_TENSOR
    assert O.rel_err(as_f32(y), ref_matmul(x, w.T)) <= 1e-2


def test_mixed_dtype_extension_through_tensor():
    rng = np.random.default_rng(2)
    a = rng.integers(-127, 128, size=(128, 256), dtype=np.int8)
    b = rng.integers(-127, 128, size=(256, 128), dtype=np.int8)
    r = Tensor.from_torch(torch.from_numpy(a).to(DEV)).matmul(Tensor.from_torch(torch.from_numpy(b).to(DEV)),
                                                               out_dtype=DType.I32)
    assert np.array_equal(r.to_torch().cpu().numpy(), a.astype(np.int32) @ b.astype(np.int32))
    x = np.clip(rng.standard_normal((128, 256)).astype(np.float32) * 64, -448, 448)
    xt = Tensor.from_torch(torch.from_numpy(x).to(DEV)).to_dtype(DType.F8E4M3)
    assert np.array_equal(xt.storage.view(torch.uint8).cpu().numpy(), O.f32_to_e4m3(x).reshape(-1))
    r = xt.matmul(xt.transpose(0, 1), out_dtype=DType.BF16, scale_lhs=1 / 64, scale_rhs=1 / 64)
    xf = O.e4m3_to_f32(O.f32_to_e4m3(x))
    assert O.rel_err(as_f32(r), np.matmul(xf, xf.T) / 4096) <= 6e-2


def test_to_dtype_round_trip():
    rng = np.random.default_rng(3)
    x = rng.standard_normal((33, 65)).astype(np.float32)
    t = Tensor.from_torch(torch.from_numpy(x).to(DEV))
    for dt, code in ((DType.BF16, O.BF16), (DType.F16, O.F16)):
        n = t.transpose(0, 1).to_dtype(dt)                 # strided source
        assert n.shape == (65, 33)
        assert np.array_equal(from_dev(n.storage.view(torch.int16), code), O.narrow(x.T.copy(), code).reshape(-1))
        back = n.to_dtype(DType.F32)
        assert np.array_equal(back.to_torch().cpu().numpy(), O.widen(O.narrow(x.T.copy(), code), code))


@pytest.mark.parametrize("in_dt,out_dt", [(O.BF16, O.BF16), (O.I8, O.I32), (O.F8E4M3, O.BF16)])
def test_host_buffer_forms_match_device_forms(in_dt, out_dt):
    """hodu_b200_matmul_host / dot_host: pinned host operands in, host result out."""
    rng = np.random.default_rng(4 + in_dt)

    def storage(shape):
        if in_dt == O.I8:
            return rng.integers(-127, 128, size=shape, dtype=np.int8)
        return O.narrow(rng.standard_normal(shape).astype(np.float32) * (8 if in_dt == O.F8E4M3 else 1), in_dt)

    def pinned(a):
        t = torch.from_numpy(np.ascontiguousarray(a).view(np.uint8).reshape(-1).copy()).pin_memory()
        return t

    # the fourth and fifth cases have a rhs of 8 MiB or more: it travels in column panels, with
    # a narrower last panel and a short last row block; in the fifth the lhs is a batch of three
    k_big = 4096 // np.dtype(O.NP_STORAGE[in_dt]).itemsize
    cases = [("dot", (1000, 256), (256, 384)), ("matmul", (5, 136, 128), (5, 128, 72)), ("matmul", (3, 200, 64), (64, 40)),
             ("dot", (700, k_big), (k_big, 2432)), ("matmul", (3, 200, k_big), (k_big, 2048))]
    for kind, ls, rs in cases:
        a, b = storage(ls), storage(rs)
        la, lb = Layout.from_shape(ls), Layout.from_shape(rs)
        if kind == "dot":
            md, out_shape = dot_metadata(la, lb), (ls[0], rs[1])
        else:
            out_shape = (ls[0], ls[1], rs[-1])
            md = matmul_metadata(la, lb, Layout.from_shape(out_shape))
        n_out = int(np.prod(out_shape))
        pa, pb = pinned(a), pinned(b)
        po = torch.empty(n_out * np.dtype(O.NP_STORAGE[out_dt]).itemsize, dtype=torch.uint8).pin_memory()
        scales = (0.5, 2.0) if in_dt == O.F8E4M3 else (1.0, 1.0)
        K.call_ops_matmul_host(DType(in_dt), DType(out_dt), 0, pa.data_ptr(), pb.data_ptr(), po.data_ptr(), md,
                               scales[0], scales[1], is_dot=(kind == "dot"))
        assert K.last_status(0) == 0
        got = po.numpy().view(O.NP_STORAGE[out_dt])
        want = O.matmul(a, b, md, in_dt, out_dt, scales[0] * scales[1], is_dot=(kind == "dot"))
        if out_dt == O.I32:
            assert np.array_equal(got, want)
        else:
            assert O.rel_err(O.widen(got, out_dt), O.widen(want, out_dt)) <= (6e-2 if in_dt == O.F8E4M3 else 1e-2)
    # non-contiguous host operands are refused, not silently copied
    with pytest.raises(Exception):
        K.call_ops_matmul_host(DType(in_dt), DType(out_dt), 0, pa.data_ptr(), pb.data_ptr(), po.data_ptr(),
                               dot_metadata(Layout((4, 4), (1, 4), 0), Layout.from_shape((4, 4))), is_dot=True)


def test_bounded_wait_reports_through_the_status_word():
    """A wait nothing satisfies gives up after its limit; the kernel returns normally, the
    status word says so, and the context keeps working."""
    lib = _lib.lib()
    assert K.last_status(0) == 0
    assert lib.hodu_b200_debug_wait_timeout(0, None, 50) == 0
    with pytest.raises(Exception) as e:
        K.last_status(0)
    assert "device status" in str(e.value)
    assert K.last_status(0) == 0  # reading cleared it
    a = O.f32_to_bf16(np.ones((128, 64), np.float32))
    md = dot_metadata(Layout.from_shape((128, 64)), Layout.from_shape((64, 128)))
    ta = to_dev(a)
    out = torch.empty(128 * 128, dtype=torch.int16, device=DEV)
    K.force_path(_lib.PATH_TENSOR)
    try:
        K.call_ops_dot(K.dot.BF16, 0, ta.data_ptr(), ta.data_ptr(), out.data_ptr(), md, 0)
    finally:
        K.force_path(_lib.PATH_AUTO)
    assert K.last_status(0) == 0
    assert np.all(O.widen(from_dev(out, O.BF16), O.BF16) == 64.0)


def test_concurrent_calls_from_several_threads_on_one_device():
    """`call_ops_matmul` may be called from any thread, two threads at once on the same device
    (the reference's `Kernels` / device pool are RwLock-guarded maps: src/kernel.rs:102-107).
    Four threads, each on its own stream, alternate two shapes so that tensor-map encoding, the
    per-instantiation launch set-up and the scratch pool are all hit concurrently."""
    import threading
    import torch
    from hodu_b200 import kernels as K
    from hodu_b200.layout import Layout
    from hodu_b200.op_metadatas import dot_metadata
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(1)
    shapes = [(512, 384, 256, torch.bfloat16, K.dot.BF16), (256, 512, 384, torch.float32, K.dot.F32)]
    data = []
    for m, k, n, dt, kern in shapes:
        a = torch.randn(m, k, generator=g, device=dev).to(dt)
        b = torch.randn(k, n, generator=g, device=dev).to(dt)
        out = torch.empty(m * n, dtype=dt, device=dev)
        K.call_ops_dot(kern, 0, a.data_ptr(), b.data_ptr(), out.data_ptr(),
                       dot_metadata(Layout.from_shape((m, k)), Layout.from_shape((k, n))), 0)
        torch.cuda.synchronize()
        data.append((a, b, out.clone()))
    errors = []

    def worker(tid):
        try:
            s = torch.cuda.Stream(device=dev)
            for it in range(40):
                m, k, n, dt, kern = shapes[(tid + it) % 2]
                a, b, want = data[(tid + it) % 2]
                out = torch.empty(m * n, dtype=dt, device=dev)
                K.call_ops_dot(kern, 0, a.data_ptr(), b.data_ptr(), out.data_ptr(),
                               dot_metadata(Layout.from_shape((m, k)), Layout.from_shape((k, n))), s.cuda_stream)
                if K.last_path() != _lib.PATH_TENSOR:   # a fresh thread must not fall back silently
                    errors.append(f"thread {tid} iteration {it}: path {K.last_path()} instead of the tensor-core kernel")
                    return
                s.synchronize()
                if not torch.equal(out, want):
                    d = (out != want).reshape(m, n)
                    rows, cols = d.any(1).nonzero().flatten().tolist(), d.any(0).nonzero().flatten().tolist()
                    errors.append(f"thread {tid} iteration {it} ({m}x{k}x{n}): {int(d.sum())} elements differ from the "
                                  f"single-threaded result; rows {rows[:2]}..{rows[-2:]} ({len(rows)}), "
                                  f"cols {cols[:2]}..{cols[-2:]} ({len(cols)}), "
                                  f"max |diff| {(out.float() - want.float()).abs().max().item():.3g}")
                    return
        except Exception as e:  # noqa: BLE001
            errors.append(f"thread {tid}: {e!r}")

    threads = [threading.Thread(target=worker, args=(t,)) for t in range(4)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    assert K.last_status(0) == 0


def test_shutdown_releases_everything_and_the_next_call_sets_up_again():
    """`hodu_b200_shutdown` frees the status word, the scratch pool, the host-pipeline staging and
    streams; the next call on the device initialises them again and computes the same result."""
    lib = _lib.lib()
    rng = np.random.default_rng(21)
    a = rng.standard_normal((300, 1024)).astype(np.float32)     # f32: goes through the scratch pool
    b = rng.standard_normal((1024, 200)).astype(np.float32)
    md = dot_metadata(Layout.from_shape(a.shape), Layout.from_shape(b.shape))
    ta, tb = to_dev(a), to_dev(b)
    out1 = torch.empty(300 * 200, dtype=torch.float32, device=DEV)
    K.call_ops_dot(K.dot.F32, 0, ta.data_ptr(), tb.data_ptr(), out1.data_ptr(), md, 0)
    pa = torch.from_numpy(a.reshape(-1).copy()).pin_memory()
    pb = torch.from_numpy(b.reshape(-1).copy()).pin_memory()
    po = torch.empty(300 * 200, dtype=torch.float32).pin_memory()
    K.call_ops_matmul_host(DType.F32, DType.F32, 0, pa.data_ptr(), pb.data_ptr(), po.data_ptr(), md, is_dot=True)
    assert K.last_status(0) == 0
    free_before = torch.cuda.mem_get_info(0)[0]
    lib.hodu_b200_shutdown(0)
    lib.hodu_b200_shutdown(0)                                   # idempotent
    assert torch.cuda.mem_get_info(0)[0] >= free_before         # nothing was kept
    assert lib.hodu_b200_init(0) == 0
    out2 = torch.empty(300 * 200, dtype=torch.float32, device=DEV)
    K.call_ops_dot(K.dot.F32, 0, ta.data_ptr(), tb.data_ptr(), out2.data_ptr(), md, 0)
    K.call_ops_matmul_host(DType.F32, DType.F32, 0, pa.data_ptr(), pb.data_ptr(), po.data_ptr(), md, is_dot=True)
    assert K.last_status(0) == 0
    assert torch.equal(out1, out2)
    assert O.rel_err(po.numpy(), O.matmul(a, b, md, O.F32, is_dot=True)) <= 1e-4
