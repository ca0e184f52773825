"""Helpers for the GPU parity tests: move raw storage to the device with torch, call the
library through its C ABI (hodu_b200.kernels -> ctypes), bring raw storage back."""
import numpy as np
import torch

from hodu_b200 import kernels as K
from hodu_b200.dtype import DType
from oracle import oracle as O

DEV = torch.device("cuda:0")
TORCH_STORAGE = {O.F8E4M3: torch.uint8, O.BF16: torch.int16, O.F16: torch.int16, O.F32: torch.float32,
                 O.I8: torch.int8, O.I32: torch.int32}


def to_dev(bits: np.ndarray) -> torch.Tensor:
    a = np.ascontiguousarray(bits).reshape(-1)
    if a.dtype == np.uint16:
        a = a.view(np.int16)
    return torch.from_numpy(a).to(DEV)


def from_dev(t: torch.Tensor, dtype: int) -> np.ndarray:
    return t.cpu().numpy().view(O.NP_STORAGE[dtype])


def new_out(n: int, dtype: int, canary: int = 64) -> torch.Tensor:
    """Output buffer of n elements followed by `canary` elements of a known pattern."""
    t = torch.empty(n + canary, dtype=TORCH_STORAGE[dtype], device=DEV)
    t.view(torch.uint8).fill_(0xA5)
    return t


def canary_intact(t: torch.Tensor, n: int) -> bool:
    tail = t[n:].view(torch.uint8)
    return bool((tail == 0xA5).all().item())


def gpu_matmul(lhs_bits, rhs_bits, md, in_dt, out_dt=None, scales=(1.0, 1.0), is_dot=False, path=K._lib.PATH_AUTO,
               plain_api=False):
    """Runs one call; returns (raw output storage, path taken).  Checks the canary and the
    device status word."""
    out_dt = in_dt if out_dt is None else out_dt
    ta, tb = to_dev(lhs_bits), to_dev(rhs_bits)
    n_out = int(md[0]) * int(md[2]) if is_dot else int(md[0])
    out = new_out(n_out, out_dt)
    prev = K.force_path(path)
    try:
        if plain_api:
            fam = K.dot if is_dot else K.matmul
            call = K.call_ops_dot if is_dot else K.call_ops_matmul
            call(getattr(fam, str(DType(in_dt)).upper()), 0, ta.data_ptr(), tb.data_ptr(), out.data_ptr(), md, 0)
        else:
            K.call_ops_matmul_ex(DType(in_dt), DType(out_dt), 0, ta.data_ptr(), tb.data_ptr(), out.data_ptr(), md,
                                 scales[0], scales[1], 0, is_dot=is_dot)
        taken = K.last_path()
    finally:
        K.force_path(prev)
    assert K.last_status(0) == 0
    assert canary_intact(out, n_out), "kernel wrote past the end of the output"
    return from_dev(out[:n_out], out_dt), taken


def check_close(got_bits, want_bits, out_dt, tol):
    """Bit-exact for integer outputs; max|got-want| / max|want| <= tol for floating ones."""
    if out_dt in (O.I32, O.I8):
        assert np.array_equal(got_bits, want_bits), f"{int((got_bits != want_bits).sum())} integer mismatches"
        return 0.0
    err = O.rel_err(O.widen(got_bits, out_dt), O.widen(want_bits, out_dt))
    assert err <= tol, f"relative error {err:.3e} > {tol}"
    return err
