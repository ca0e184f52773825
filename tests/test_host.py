"""Host-side logic and the C-ABI surface; no GPU needed (no compute call is made)."""
import ctypes
import os
import re

import numpy as np
import pytest

from hodu_b200 import CudaKernelError, DType, Layout, _lib, kernels
from hodu_b200.op_metadatas import cast_metadata, dot_metadata, matmul_metadata, swiglu_metadata

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol(built_lib):
    header = open(os.path.join(ROOT, "include", "hodu_b200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(hodu_b200_\w+)\s*\(", header))
    assert len(declared) >= 15
    for name in sorted(declared):
        assert hasattr(built_lib, name), f"{name} is declared in the header but not exported"
    assert declared == set(_lib.SIGNATURES), "ctypes signature table and header disagree"
    assert built_lib.hodu_b200_version() == 100


def test_dtype_codes_match_reference_enum():
    want = {"BOOL": 0, "F8E4M3": 1, "F8E5M2": 2, "BF16": 3, "F16": 4, "F32": 5, "F64": 6, "U8": 7, "U16": 8,
            "U32": 9, "U64": 10, "I8": 11, "I16": 12, "I32": 13, "I64": 14}
    assert {d.name: int(d) for d in DType} == want
    assert str(DType.F8E4M3) == "f8e4m3" and str(DType.BF16) == "bf16"
    assert kernels.matmul.BF16.name == "hodu_cuda_matmul_bf16"
    assert kernels.dot.F32.name == "hodu_cuda_dot_f32"
    assert kernels.cast.F32_BF16.name == "hodu_cuda_cast_f32_to_bf16"


def test_layout_views():
    l = Layout.from_shape((4, 6, 8))
    assert l.strides == (48, 8, 1) and l.is_contiguous() and l.size() == 192
    t = l.transpose(-2, -1)
    assert t.shape == (4, 8, 6) and t.strides == (48, 1, 8) and not t.is_contiguous()
    b = Layout.from_shape((1, 6, 8)).broadcast_to((5, 6, 8))
    assert b.strides == (0, 8, 1)
    b2 = Layout.from_shape((6, 8)).broadcast_to((2, 3, 6, 8))
    assert b2.strides == (0, 0, 8, 1)
    with pytest.raises(ValueError):
        Layout.from_shape((2, 6, 8)).broadcast_to((5, 6, 8))
    assert Layout.from_shape((3, 1, 7)).is_contiguous()
    assert Layout((3, 1, 7), (7, 999, 1)).is_contiguous()  # extent-1 dims do not matter


def test_metadata_wire_formats():
    # the reference's own hand-built vectors (crates/hodu_cuda_kernels/tests/ops_matrix.rs:52-101,189-262)
    assert matmul_metadata(Layout.from_shape((2, 3)), Layout.from_shape((3, 2)), Layout.from_shape((2, 2))) == \
        [4, 2, 2, 0, 2, 3, 3, 2, 3, 1, 2, 1, 0, 0, 2, 3, 2]
    assert matmul_metadata(Layout.from_shape((2, 2, 3)), Layout.from_shape((3, 2)), Layout.from_shape((2, 2, 2))) == \
        [8, 3, 2, 1, 2, 2, 3, 3, 2, 2, 6, 3, 1, 2, 1, 0, 0, 2, 3, 2]
    assert dot_metadata(Layout.from_shape((2, 3)), Layout.from_shape((3, 2))) == [2, 3, 2, 3, 1, 2, 1, 0, 0]
    # Linear: weight [N,K] passed as a transposed view -> rhs strides (1, K)
    w = Layout.from_shape((5, 3)).transpose(-2, -1)
    assert dot_metadata(Layout.from_shape((2, 3)), w) == [2, 3, 5, 3, 1, 1, 3, 0, 0]
    assert cast_metadata(Layout((2, 3), (1, 2), 4)) == [6, 2, 2, 3, 1, 2, 4]
    assert len(swiglu_metadata(Layout.from_shape((4, 8)), w.__class__.from_shape((8, 6)), Layout.from_shape((8, 6)))) == 12
    with pytest.raises(ValueError):
        matmul_metadata(Layout.from_shape((2, 3)), Layout.from_shape((4, 2)), Layout.from_shape((2, 2)))
    with pytest.raises(ValueError):
        matmul_metadata(Layout.from_shape((2, 4, 3)), Layout.from_shape((3, 3, 2)), Layout.from_shape((2, 4, 2)))


def _expect(code_kind, fn, *args):
    with pytest.raises(CudaKernelError) as e:
        fn(*args)
    assert e.value.kind == code_kind, e.value


def test_error_codes_without_touching_a_device(built_lib):
    """Argument errors are reported before any CUDA call, with the reference's error variants."""
    good_md = [4, 2, 2, 0, 2, 3, 3, 2, 3, 1, 2, 1, 0, 0, 2, 3, 2]
    # metadata too short / wrong length
    _expect("invalid input", kernels.call_ops_matmul, kernels.matmul.F32, 0, 1, 1, 1, good_md[:-1])
    _expect("invalid input", kernels.call_ops_dot, kernels.dot.F32, 0, 1, 1, 1, [2, 3, 2, 3, 1, 2, 1, 0])
    # M,K,N disagreeing with the shapes
    bad = list(good_md); bad[-1] = 5
    _expect("invalid input", kernels.call_ops_matmul, kernels.matmul.F32, 0, 1, 1, 1, bad)
    # num_els wrong
    bad = list(good_md); bad[0] = 5
    _expect("invalid input", kernels.call_ops_matmul, kernels.matmul.F32, 0, 1, 1, 1, bad)
    # batch dim that does not broadcast
    md = matmul_metadata(Layout.from_shape((2, 2, 3)), Layout.from_shape((3, 2)), Layout.from_shape((2, 2, 2)))
    md[4] = 3
    _expect("invalid input", kernels.call_ops_matmul, kernels.matmul.F32, 0, 1, 1, 1, md)
    # unsupported dtypes are an error, never a fallback
    _expect("invalid kernel", kernels.call_ops_matmul, kernels.matmul.F64, 0, 1, 1, 1, good_md)
    _expect("invalid kernel", kernels.call_ops_matmul, kernels.Kernel("hodu_cuda_matmul_u8"), 0, 1, 1, 1, good_md)
    _expect("invalid kernel", kernels.call_ops_matmul, kernels.Kernel("hodu_cuda_nonsense"), 0, 1, 1, 1, good_md)
    _expect("invalid kernel", kernels.call_ops_matmul_ex, DType.BF16, DType.I32, 0, 1, 1, 1, good_md)
    # null pointers
    _expect("invalid input", kernels.call_ops_matmul, kernels.matmul.F32, 0, 0, 1, 1, good_md)
    # integer matmul takes no scale
    _expect("invalid input", kernels.call_ops_matmul_ex, DType.I8, DType.I32, 0, 1, 1, 1, good_md, 0.5, 1.0)
    # device id out of range
    _expect("device not initialised", kernels.call_ops_matmul, kernels.matmul.F32, 99, 1, 1, 1, good_md)
    # swiglu metadata length
    _expect("invalid input", kernels.call_ops_swiglu, DType.BF16, 0, 1, 1, 1, 1, [1, 2, 3])
    # empty problems succeed without a device: nothing to compute
    empty = matmul_metadata(Layout.from_shape((0, 3)), Layout.from_shape((3, 2)), Layout.from_shape((0, 2)))
    kernels.call_ops_matmul(kernels.matmul.F32, 0, 0, 0, 0, empty)
    assert built_lib.hodu_b200_strerror(-3) == b"launch error"


def test_cast_metadata_errors(built_lib):
    _expect("invalid input", kernels.call_ops_cast, kernels.cast.F32_BF16, 0, 1, 1, [4, 1, 4, 1])       # too short
    _expect("invalid input", kernels.call_ops_cast, kernels.cast.F32_BF16, 0, 1, 1, [5, 1, 4, 1, 0])    # num_els != shape
    _expect("invalid input", kernels.call_ops_cast, kernels.cast.F32_BF16, 0, 0, 1, [4, 1, 4, 1, 0])    # null input
    _expect("invalid kernel", kernels.call_ops_cast, kernels.cast.F32_I64, 0, 1, 1, [4, 1, 4, 1, 0])    # pair not offered
    _expect("device not initialised", kernels.call_ops_cast, kernels.cast.F32_BF16, 99, 1, 1, [4, 1, 4, 1, 0])
    kernels.call_ops_cast(kernels.cast.F32_BF16, 0, 0, 0, [0, 1, 0, 1, 0])                                # empty: nothing to do


def test_shard_range_covers_everything():
    from hodu_b200.dist import shard_range
    for total in (0, 1, 7, 16, 8192, 16385):
        for world in (1, 2, 3, 4, 8):
            spans = [shard_range(total, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_range(4, 4, 4)


def test_synthetic_inputs_are_seeded_and_shaped():
    from hodu_b200 import synthetic as S
    a = S.config2(scale=64, batches=2)
    b = S.config2(scale=64, batches=2)
    assert a["a"].shape == (2, 32, 32) and np.array_equal(a["a"], b["a"]) and not np.array_equal(a["a"], a["b"])
    c3 = S.config3(scale=256)
    assert np.abs(c3["a"]).max() <= 448 and c3["a"].dtype == np.float32
    c4 = S.config4(scale=256)
    assert c4["a"].dtype == np.int8 and c4["a"].min() >= -127
    c5 = S.config5(scale=128)
    assert c5["w_gate"].shape == (32, 112) and c5["w_down"].shape == (112, 32)
    assert S.FLOPS[2] == 274877906944 and S.FLOPS[3] == 1099511627776 and S.FLOPS[5] == 5772436045824


# ---------------------------------------------------------------- einsum equation parser
# Mirrors the parser tests of the reference (crates/hodu_core/src/einsum.rs:171-244).
def test_einsum_parse_forms():
    from hodu_b200.einsum import ParsedEinsum, einsum_metadata
    p = ParsedEinsum.parse("ij,jk->ik", [(2, 3), (3, 4)])
    assert p.input_subscripts == [["i", "j"], ["j", "k"]] and p.output_subscripts == ["i", "k"]
    assert p.contraction_indices == ["j"] and p.compute_output_shape() == [2, 4]
    p = ParsedEinsum.parse("ij->ji", [(2, 3)])
    assert p.output_subscripts == ["j", "i"] and p.contraction_indices == [] and p.compute_output_shape() == [3, 2]
    p = ParsedEinsum.parse("ii->", [(3, 3)])
    assert p.output_subscripts == [] and p.contraction_indices == ["i"]
    p = ParsedEinsum.parse("i,j->ij", [(3,), (4,)])
    assert p.contraction_indices == [] and p.compute_output_shape() == [3, 4]
    p = ParsedEinsum.parse("bij,bjk->bik", [(2, 3, 4), (2, 4, 5)])
    assert p.contraction_indices == ["j"] and p.compute_output_shape() == [2, 3, 5]
    p = ParsedEinsum.parse("ij,jk", [(2, 3), (3, 4)])   # implicit output: indices that occur once
    assert p.output_subscripts == ["i", "k"]
    with pytest.raises(ValueError):
        ParsedEinsum.parse("ij,jk->ik", [(2, 3), (4, 5)])
    with pytest.raises(ValueError):
        ParsedEinsum.parse("ij,jk->ik", [(2, 3)])
    with pytest.raises(ValueError):
        ParsedEinsum.parse("ij->iz", [(2, 3)])
    # wire format of "ij,jk->ik" as the reference's test helper builds it
    # (crates/hodu_cpu_kernels/tests/ops_einsum.rs:18-84)
    p = ParsedEinsum.parse("ij,jk->ik", [(2, 3), (3, 4)])
    md = einsum_metadata(p, [Layout.from_shape((2, 3)), Layout.from_shape((3, 4))], Layout.from_shape((2, 4)))
    assert md == [8, 2, 3, 1, 2, 2, 4,  2, 2, 3, 3, 1, 0, 0, 1,  2, 3, 4, 4, 1, 0, 1, 2,  1,  2, 3, 4,  0, 2]


def _einsum_md(eq, shapes):
    from hodu_b200.einsum import ParsedEinsum, einsum_metadata
    p = ParsedEinsum.parse(eq, shapes)
    return einsum_metadata(p, [Layout.from_shape(s) for s in shapes],
                           Layout.from_shape(tuple(p.compute_output_shape())))


@pytest.mark.parametrize("eq,shapes", [("ii->", [(3, 3)]), ("ij->ji", [(2, 3)]), ("ij,jk->", [(2, 3), (3, 4)]),
                                        ("ij,jk,kl->il", [(2, 3), (3, 4), (4, 5)]), ("bij,bjk->ibk", [(2, 3, 4), (2, 4, 5)]),
                                        ("ii,ij->j", [(3, 3), (3, 2)])])
def test_einsum_forms_that_are_not_matrix_products_are_refused(built_lib, eq, shapes):
    md = _einsum_md(eq, shapes)
    with pytest.raises(CudaKernelError) as e:   # refused while parsing: no device is touched
        kernels.call_ops_einsum(kernels.einsum.F32, 0, [0x1000] * len(shapes), 0x2000, md)
    assert e.value.code == -1


def test_einsum_and_linear_argument_errors(built_lib):
    md = _einsum_md("ij,jk->ik", [(2, 3), (3, 4)])
    with pytest.raises(CudaKernelError) as e:
        kernels.call_ops_einsum(kernels.einsum.F32, 0, [0x1000, 0x1000], 0x2000, md[:-1])
    assert e.value.code == -2
    with pytest.raises(CudaKernelError) as e:
        kernels.call_ops_einsum(kernels.einsum.F64, 0, [0x1000, 0x1000], 0x2000, md)
    assert e.value.code == -1
    mm = matmul_metadata(Layout.from_shape((4, 8)), Layout.from_shape((8, 2)), Layout.from_shape((4, 2)))
    with pytest.raises(CudaKernelError) as e:
        kernels.call_ops_linear(DType.BF16, 0, 0x1000, 0x1000, 0x1000, 0x2000, [*mm, 1, 0], flags=7)
    assert e.value.code == -2
    with pytest.raises(CudaKernelError) as e:
        kernels.call_ops_linear(DType.I8, 0, 0x1000, 0x1000, 0x1000, 0x2000, [*mm, 1, 0])
    assert e.value.code == -1


def test_bench_reference_arm_prints_the_contract_line():
    """`bench.py --impl reference` needs no GPU: one JSON line with the contract's keys."""
    import json
    import subprocess
    import sys
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--workload", "c1",
                          "--steps", "2", "--warmup", "1"], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-500:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better",
                "scaling", "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e", "gpu_launches"):
        assert key in line, key
    assert line["impl"] == "reference" and line["unit"] == "TFLOP/s" and line["value"] > 0
    assert line["cpu_baseline"]["kind"] in ("reference", "port") and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["gpu_launches"] == 0
