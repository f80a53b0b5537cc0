"""CPU-side checks of the C-ABI library: it loads without a GPU, exports every symbol that
include/mcb.h declares, refuses to create a context when no device exists (no CPU fallback),
and its host-only helper works."""
import ctypes as C
import os
import re
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from modernchainer_b200 import _lib, build
    if not os.path.exists(_lib.LIB_PATH):
        build.build()
    return _lib.load()


def test_every_declared_symbol_is_exported(lib):
    from modernchainer_b200 import _lib
    protos = _lib.parse_header()
    assert len(protos) > 100
    declared = set(re.findall(r"\b(mcb_[a-z0-9_]+)\s*\(", open(_lib.HEADER).read()))
    declared -= {"mcb_status"}
    for name in declared:
        assert hasattr(lib, name), name
        assert name in protos, name


def test_no_cpu_fallback_without_device(lib):
    if lib.mcb_device_count() > 0:
        pytest.skip("a GPU is present")
    h = C.c_void_p()
    assert lib.mcb_ctx_create(0, C.byref(h)) == 8  # MCB_BACKEND
    import modernchainer_b200 as mc
    with pytest.raises(mc.McbError):
        mc.Context(0)


def test_product_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "modernchainer_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
                text = open(os.path.join(dirpath, f), errors="ignore").read()
                assert "oracle" not in text.lower().replace("oracle/", "oracle/") or "import oracle" not in text, f
                assert "mc_oracle" not in text, f
                assert "from oracle" not in text and "import oracle" not in text, f


def test_bucket_planner(lib):
    sizes = np.array([10, 20, 30, 40, 50], np.int64)
    out = np.zeros(5, np.int32)
    nb = C.c_int32()
    st = lib.mcb_dp_plan_buckets(sizes.ctypes.data_as(C.c_void_p), 5, 60, out.ctypes.data_as(C.c_void_p), C.byref(nb))
    assert st == 0
    # walked from the last tensor (first gradient ready in backward) to the first
    assert out.tolist() == [2, 2, 2, 1, 0] and nb.value == 3
    st = lib.mcb_dp_plan_buckets(sizes.ctypes.data_as(C.c_void_p), 5, 1000, out.ctypes.data_as(C.c_void_p), C.byref(nb))
    assert out.tolist() == [0] * 5 and nb.value == 1
    st = lib.mcb_dp_plan_buckets(sizes.ctypes.data_as(C.c_void_p), 5, 1, out.ctypes.data_as(C.c_void_p), C.byref(nb))
    assert out.tolist() == [4, 3, 2, 1, 0] and nb.value == 5
    assert lib.mcb_dp_plan_buckets(sizes.ctypes.data_as(C.c_void_p), 5, 0, out.ctypes.data_as(C.c_void_p), C.byref(nb)) == 5


def test_host_bf16_helpers_match_oracle(oracle):
    import modernchainer_b200 as mc
    x = np.random.default_rng(0).standard_normal(4096).astype(np.float32) * 3
    assert np.array_equal(mc.f32_to_bf16_bits(x), oracle.f32_to_bf16_bits(x))
    assert np.array_equal(mc.bf16_bits_to_f32(mc.f32_to_bf16_bits(x)), oracle.round_bf16(x))


def test_lr_schedules_match_the_oracle_restatement():
    """The schedules are host functions of the step (optim/src/lib.rs:245-326): the library's C entry
    points against the oracle's restatement, bit for bit, including the edge cases the formulas carry
    (zero warm-up, step past the end, step_size 0, total_steps 0)."""
    import modernchainer_b200 as mc
    from oracle import ref as oracle
    steps = [0, 1, 2, 9, 10, 11, 99, 100, 101, 5000]
    for args in [(10, 100, 1e-3, 1e-5), (0, 100, 3e-4, 0.0), (10, 10, 1e-3, 1e-4)]:
        a, b = mc.LinearWarmupCosineLR(*args), oracle.LinearWarmupCosineLR(*args)
        for s in steps:
            assert a.get_lr(s) == b.get_lr(s), (args, s)
    for args in [(0.1, 30, 0.5), (0.1, 0, 0.9), (1.0, 1, 1.1)]:
        a, b = mc.StepLR(*args), oracle.StepLR(*args)
        for s in steps:
            assert a.get_lr(s) == b.get_lr(s), (args, s)
    for args in [(1e-3, 100, 2.0, 1e-5), (1e-3, 0, 0.5, 0.0), (1e-3, 100, 1.0, 1e-4)]:
        a, b = mc.PolynomialLR(*args), oracle.PolynomialLR(*args)
        for s in steps:
            ga, gb = a.get_lr(s), b.get_lr(s)
            assert ga == gb or abs(ga - gb) <= 1e-15 * abs(gb), (args, s)  # pow() of two C libraries: last-bit room
    assert mc.ConstantLR(0.3).get_lr(17) == 0.3


def test_chainer_facade_imports_without_a_gpu_and_refuses_to_compute():
    """The facade package loads on a host without a GPU (host-side Tensor and initialiser work), but the
    first Variable needs the device context and fails loudly: there is no CPU execution path."""
    import ctypes as C
    import modernchainer_b200.chainer as chainer
    import modernchainer_b200.chainer.functions as F
    import modernchainer_b200.chainer.links as L
    import modernchainer_b200.chainer.optimizers as O
    from oracle import ref as oracle
    assert chainer.__version__ and chainer.vulkan_available() is False
    t = chainer.Tensor.from_list([1.0, 2.0, 3.0, 4.0], [2, 2])
    assert t.shape == [2, 2] and t.dtype == "f32" and t.device == "cpu" and t.astype("i64").dtype == "i64"
    assert set(F.__all__) >= {"linear", "softmax_cross_entropy", "permute", "transpose"} and "Linear" in L.__all__ and "AdamW" in O.__all__
    # the initialiser behind the links is the reference's generator: bit-identical to the oracle's restatement
    for shape, fan_in, seed in [((3, 5), 5, 0), ((100, 784), 784, 0), ((64, 3, 3, 3), 27, 7), ((7,), 1, 123456789)]:
        out = np.empty(int(np.prod(shape)), np.float32)
        assert chainer._api._lib.load().mcb_he_normal(out.ctypes.data_as(C.c_void_p), out.size, fan_in, seed) == 0
        assert np.array_equal(out.reshape(shape), oracle.he_normal(shape, fan_in, seed))
    if not chainer.cuda_available():
        with pytest.raises(Exception):
            chainer.Variable(t)


def test_rust_mirror_matches_the_header():
    """include/mcb_sys.rs is generated from include/mcb.h: the committed file is what the generator gives today,
    it declares every function of the header exactly once, and every mcb_* call in the hand-written trait
    forwarding (include/mcb_ops.rs) names a declared function and passes as many arguments as the header lists.
    All ten status codes appear in the status -> core::Error map."""
    import re
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    gen = os.path.join(root, "include", "gen_rust_binding.py")
    assert subprocess.run([sys.executable, gen, "--check"]).returncode == 0
    from modernchainer_b200 import _lib
    protos = _lib.parse_header()
    sys_rs = open(os.path.join(root, "include", "mcb_sys.rs")).read()
    declared = re.findall(r"pub fn (mcb_\w+)\(([^)]*)\)", sys_rs)
    assert sorted(n for n, _ in declared) == sorted(protos)
    arity = {n: (0 if not a.strip() else a.count(":")) for n, a in declared}
    for n, (_, argtypes) in protos.items():
        assert arity[n] == len(argtypes), n
    ops_rs = open(os.path.join(root, "include", "mcb_ops.rs")).read()
    ops_rs = re.sub(r"//[^\n]*", "", ops_rs)
    calls = 0
    for m in re.finditer(r"\b(mcb_[a-z0-9_]+)\s*\(", ops_rs):
        name = m.group(1)
        assert name in arity, name
        depth, i, args, cur = 1, m.end(), 0, ""
        while depth:
            ch = ops_rs[i]
            if ch in "([{":
                depth += 1
            elif ch in ")]}":
                depth -= 1
            elif ch == "," and depth == 1:
                args += 1
                cur = ""
                i += 1
                continue
            cur += ch
            i += 1
        args += 1 if cur.strip(" \n)") or args else 0
        assert args == arity[name], (name, args, arity[name])
        calls += 1
    assert calls >= 25
    for code in ("MCB_OK", "MCB_SHAPE_MISMATCH", "MCB_BROADCAST", "MCB_DTYPE_MISMATCH", "MCB_UNSUPPORTED_DTYPE", "MCB_INVALID_ARGUMENT",
                 "MCB_OUT_OF_BOUNDS", "MCB_UNSUPPORTED", "MCB_IO"):
        assert re.search(code + r"\s*=>", ops_rs), code
    assert "Error::Backend" in ops_rs
