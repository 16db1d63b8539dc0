"""Host-side logic that needs no GPU: the C ABI loads and exports what the header
declares, parameter validation, backend resolution, fallback bookkeeping
(reference ``tests/test_backend.py:19-131``, ``tests/test_nn_attention.py:259-340``)
and the shard arithmetic."""
import ctypes as C
import pathlib
import re
import warnings

import pytest
import torch

ROOT = pathlib.Path(__file__).resolve().parent.parent


def test_library_exports_every_declared_symbol():
    from nitrix_b200 import _cabi

    header = "".join(f.read_text() for f in sorted((ROOT / "include").glob("*.h")))
    declared = set(re.findall(r"NB200_API\s+[\w\s\*]+?\b(nb200_\w+)\s*\(", header))
    assert declared, "no NB200_API declarations parsed"
    assert declared == set(_cabi.EXPORTS)
    lib = _cabi.lib()
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.nb200_version() == _cabi.ABI_VERSION


def test_params_struct_size_matches_library():
    from nitrix_b200 import _cabi

    p = _cabi.new_params()
    p.dtype = _cabi.F32
    p.B = p.H = 1
    p.S = p.T = 4
    p.D = p.Dv = 8
    p.bh_end = 1
    kernel = C.c_int(0)
    # struct_size agrees (a mismatch is reported as INVALID with an ABI message) ...
    rc = _cabi.lib().nb200_sdpa_plan(C.byref(p), _cabi.PASS_FWD, C.byref(kernel))
    assert "ABI mismatch" not in _cabi.last_error()
    # ... and null operands are rejected, not dereferenced
    assert rc == _cabi.ERR_INVALID and "non-NULL" in _cabi.last_error()
    p.struct_size = 8
    assert _cabi.lib().nb200_sdpa_plan(C.byref(p), _cabi.PASS_FWD, C.byref(kernel)) == _cabi.ERR_INVALID
    assert "ABI mismatch" in _cabi.last_error()


def _plan(**over):
    from nitrix_b200 import _cabi

    p = _cabi.new_params()
    p.dtype = _cabi.BF16
    p.B, p.H, p.S, p.T, p.D, p.Dv = 2, 4, 256, 256, 64, 64
    for f in ("q", "k", "v", "out", "lse"):
        setattr(p, f, 0x1000)
    for f in ("q_stride", "k_stride", "v_stride", "out_stride"):
        getattr(p, f)[:] = [4 * 256 * 64, 256 * 64, 64, 1]
    p.scale = 0.125
    p.bh_end = 8
    for key, val in over.items():
        if isinstance(val, (list, tuple)):
            getattr(p, key)[:] = list(val)
        else:
            setattr(p, key, val)
    kernel = C.c_int(0)
    rc = _cabi.lib().nb200_sdpa_plan(C.byref(p), _cabi.PASS_FWD, C.byref(kernel))
    return rc, kernel.value, _cabi.last_error()


def test_plan_validation_errors():
    from nitrix_b200 import _cabi

    assert _plan(dtype=7)[0] == _cabi.ERR_INVALID
    assert _plan(D=0)[0] == _cabi.ERR_INVALID
    assert _plan(bh_end=9)[0] == _cabi.ERR_INVALID
    assert _plan(q_stride=[1, 1, 1, 2])[0] == _cabi.ERR_INVALID
    rc, kernel, _ = _plan(kernel=_cabi.KERNEL_SIMT)
    assert rc == _cabi.OK and kernel == _cabi.KERNEL_SIMT
    assert _plan(kernel=_cabi.KERNEL_SIMT, D=512, Dv=512)[0] == _cabi.ERR_UNSUPPORTED
    # fp32 is outside the tensor-core family: forcing it is a decline, not a crash
    rc, _, msg = _plan(dtype=_cabi.F32, kernel=_cabi.KERNEL_TCGEN05)
    assert rc == _cabi.ERR_UNSUPPORTED and msg


def test_backend_resolution_and_env(monkeypatch):
    from nitrix_b200 import backend as B

    monkeypatch.delenv("NITRIX_BACKEND", raising=False)
    monkeypatch.delenv("NITRIX_REPRODUCIBLE", raising=False)
    with pytest.raises(B.NitrixBackendError):
        B.resolve_backend("tpu")
    with pytest.raises(B.NitrixBackendError):
        B.resolve_backend("jax")
    monkeypatch.setenv("NITRIX_BACKEND", "bogus")
    with pytest.raises(B.NitrixBackendError):
        B.resolve_backend("auto")
    monkeypatch.setattr(B, "has_sm100_device", lambda: True)
    monkeypatch.setenv("NITRIX_BACKEND", "cuda-simt")
    assert B.resolve_backend("auto") == "cuda-simt"
    assert B.resolve_backend("cuda-sm100") == "cuda-sm100"  # keyword beats env
    monkeypatch.delenv("NITRIX_BACKEND")
    assert B.resolve_backend("auto") == "cuda-sm100"
    assert B.resolve_backend("pallas-cuda") == "cuda-sm100"
    with B.reproducible():
        assert B.resolve_backend("auto") == "cuda-simt"
        assert B.resolve_backend("cuda-sm100") == "cuda-sm100"  # explicit beats mode
    monkeypatch.setenv("NITRIX_REPRODUCIBLE", "1")
    assert B.resolve_backend("auto") == "cuda-simt"
    monkeypatch.setattr(B, "has_sm100_device", lambda: False)
    with pytest.raises(B.NitrixBackendError):  # no device: loud, never a host path
        B.resolve_backend("auto")


def test_fallback_warns_once_strict_and_silence(monkeypatch):
    from nitrix_b200 import backend as B

    monkeypatch.delenv("NITRIX_STRICT_BACKEND", raising=False)
    monkeypatch.delenv("NITRIX_SILENCE_FALLBACK", raising=False)
    B.reset_fallback_state()
    kw = dict(function="f", requested="cuda-sm100", resolved="cuda-simt", reason="r", shapes=((1, 2),), dtype="f32")
    with pytest.warns(B.NitrixBackendFallback):
        B.fallback(**kw)
    with warnings.catch_warnings():
        warnings.simplefilter("error")
        B.fallback(**kw)  # deduplicated
        B.fallback(**{**kw, "requested": "cuda-simt"})  # no change, no warning
    B.reset_fallback_state()
    with pytest.warns(B.NitrixBackendFallback):
        B.fallback(**kw)
    monkeypatch.setenv("NITRIX_SILENCE_FALLBACK", "1")
    B.reset_fallback_state()
    with warnings.catch_warnings():
        warnings.simplefilter("error")
        B.fallback(**kw)
    monkeypatch.setenv("NITRIX_STRICT_BACKEND", "1")
    with pytest.raises(B.NitrixBackendError):
        B.fallback(**kw)


def test_entry_point_validation_errors():
    from nitrix_b200.nn import attention as A

    x3 = torch.zeros(2, 4, 8)
    with pytest.raises(ValueError, match="at least 3 dims"):
        A.scaled_dot_product_attention(torch.zeros(4, 8), x3, x3)
    with pytest.raises(ValueError, match="head-dim mismatch"):
        A.scaled_dot_product_attention(x3, torch.zeros(2, 4, 6), x3)
    with pytest.raises(ValueError, match="key-length mismatch"):
        A.scaled_dot_product_attention(x3, x3, torch.zeros(2, 5, 8))


def test_own_extent_canonicalisation():
    from nitrix_b200.nn.attention import _to_own_extent

    lead, h, s, t = (2, 3), 4, 5, 6
    assert _to_own_extent(torch.zeros(4, 5, 6), lead, h, s, t).shape == (1, 4, 5, 6)
    assert _to_own_extent(torch.zeros(2, 3, 1, 1, 6), lead, h, s, t).shape == (6, 1, 1, 6)
    assert _to_own_extent(torch.zeros(2, 1, 4, 5, 6), lead, h, s, t).shape == (6, 4, 5, 6)
    assert _to_own_extent(torch.zeros(6), lead, h, s, t).shape == (1, 1, 1, 6)
    with pytest.raises(ValueError):
        _to_own_extent(torch.zeros(7), lead, h, s, t)


def test_bh_partition_covers_everything_once():
    from nitrix_b200.parallel import bh_partition, shard_axis

    for n in (0, 1, 7, 16, 128, 513):
        for w in (1, 2, 3, 4, 8):
            spans = [bh_partition(n, w, r) for r in range(w)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    assert shard_axis(32, 8, 8) == "batch" and shard_axis(1, 16, 8) == "heads" and shard_axis(3, 5, 2) == "pairs"


def test_plan_reports_the_family_that_runs():
    """The planner's three answers (no launch, no GPU needed): bf16 at head dim 64 -> tcgen05; fp32 at a head dim
    the 3 x TF32 kernels take -> the TF32 tensor path (what decides that an fp32 caller gets no fallback warning,
    as on the reference's fused path, attention.py:736-765); a head dim of 40 -> plain CUDA cores."""
    from nitrix_b200 import _cabi

    assert _plan()[:2] == (_cabi.OK, _cabi.KERNEL_TCGEN05)
    assert _plan(dtype=_cabi.F32)[:2] == (_cabi.OK, _cabi.KERNEL_MMA_TF32X3)
    # lengths need not be multiples of anything on the tensor-core family (the caller shapes the reference's docs
    # name: 217, 28, 197, 111 tokens)
    for n in (100, 217, 28, 197, 111):
        assert _plan(S=n, T=n)[:2] == (_cabi.OK, _cabi.KERNEL_TCGEN05), n
    d40 = dict(D=40, Dv=40, q_stride=[4 * 256 * 40, 256 * 40, 40, 1], k_stride=[4 * 256 * 40, 256 * 40, 40, 1],
               v_stride=[4 * 256 * 40, 256 * 40, 40, 1], out_stride=[4 * 256 * 40, 256 * 40, 40, 1])
    assert _plan(**d40)[:2] == (_cabi.OK, _cabi.KERNEL_SIMT)
    assert _plan(dtype=_cabi.F32, D=40, Dv=40, q_stride=[4 * 256 * 40, 256 * 40, 40, 1], k_stride=[4 * 256 * 40, 256 * 40, 40, 1],
                 v_stride=[4 * 256 * 40, 256 * 40, 40, 1], out_stride=[4 * 256 * 40, 256 * 40, 40, 1])[:2] == (_cabi.OK, _cabi.KERNEL_SIMT)
    # an expanded (stride 0) head axis on k is declined by the tensor-core family
    assert _plan(k_stride=[4 * 256 * 64, 0, 64, 1])[:2] == (_cabi.OK, _cabi.KERNEL_SIMT)
    # the forced family reports why it cannot take a problem
    rc, _, msg = _plan(kernel=_cabi.KERNEL_TCGEN05, **d40)
    assert rc == _cabi.ERR_UNSUPPORTED and "head dims" in msg


def test_packed_mask_and_peer_fields_are_validated():
    from nitrix_b200 import _cabi

    assert _plan(mask=0x2000, mask_stride=[0, 0, 256, 1], mask_is_bitpacked=3)[0] == _cabi.ERR_INVALID
    # a packed mask needs the tensor-core family
    rc, _, msg = _plan(mask=0x2000, mask_stride=[0, 0, 256, 1], mask_is_bitpacked=1, kernel=_cabi.KERNEL_SIMT)
    assert rc == _cabi.ERR_UNSUPPORTED and "bit-packed" in msg
    assert _plan(mask=0x2000, mask_stride=[0, 0, 256, 1], mask_is_bitpacked=1)[:2] == (_cabi.OK, _cabi.KERNEL_TCGEN05)
    assert _plan(n_out_peers=8)[0] == _cabi.ERR_INVALID
    assert _plan(n_out_peers=1)[0] == _cabi.ERR_INVALID          # out_peers[0] is NULL
    # sizes of the packed buffer: rows only / with the key-major copy / a key-only mask never needs the copy
    def pack_bytes(stride, with_t):
        p = _cabi.new_params()
        p.dtype = _cabi.BF16
        p.B, p.H, p.S, p.T, p.D, p.Dv = 2, 4, 256, 256, 64, 64
        for f in ("q", "k", "v", "out", "lse", "mask"):
            setattr(p, f, 0x1000)
        for f in ("q_stride", "k_stride", "v_stride", "out_stride"):
            getattr(p, f)[:] = [4 * 256 * 64, 256 * 64, 64, 1]
        p.mask_stride[:] = stride
        p.bh_end = 8
        n = C.c_size_t(0)
        assert _cabi.lib().nb200_mask_pack_bytes(C.byref(p), with_t, C.byref(n)) == _cabi.OK, _cabi.last_error()
        return n.value
    rows = 2 * 256 * 8 * 4                      # (B, 1, S, T) mask: 2 x 256 rows x 8 words
    assert pack_bytes([256 * 256, 0, 256, 1], 0) == rows
    assert pack_bytes([256 * 256, 0, 256, 1], 1) == 2 * rows
    assert pack_bytes([256, 0, 0, 1], 0) == pack_bytes([256, 0, 0, 1], 1) == 256 + 256   # one row + key counts


def test_backward_plan_takes_want_dbias_without_a_buffer():
    """want_dbias lets the planner and the workspace query answer for a backward with a bias gradient before the
    dbias buffer exists; a bias shared by the batch stays on tensor cores and adds an fp32 accumulator of the
    bias' own extent to the scratch."""
    from nitrix_b200 import _cabi

    def query(want):
        p = _cabi.new_params()
        p.dtype = p.bias_dtype = _cabi.BF16
        p.B, p.H, p.S, p.T, p.D, p.Dv = 2, 4, 256, 256, 128, 128
        for f in ("q", "k", "v", "out", "lse", "dout", "dq", "dk", "dv", "bias"):
            setattr(p, f, 0x1000)
        for f in ("q_stride", "k_stride", "v_stride", "out_stride", "dout_stride", "dq_stride", "dk_stride", "dv_stride"):
            getattr(p, f)[:] = [4 * 256 * 128, 256 * 128, 128, 1]
        p.bias_stride[:] = [0, 256 * 256, 256, 1]
        p.dbias_stride[:] = [4 * 256 * 256, 256 * 256, 256, 1]
        p.scale, p.bh_end, p.want_dbias = 0.1, 8, want
        kernel, need = C.c_int(0), C.c_size_t(0)
        assert _cabi.lib().nb200_sdpa_plan(C.byref(p), _cabi.PASS_BWD, C.byref(kernel)) == _cabi.OK, _cabi.last_error()
        assert _cabi.lib().nb200_sdpa_workspace_bytes(C.byref(p), _cabi.PASS_BWD, C.byref(need)) == _cabi.OK
        return kernel.value, need.value

    k0, n0 = query(0)
    k1, n1 = query(1)
    assert k0 == k1 == _cabi.KERNEL_TCGEN05
    delta = 2 * 4 * 256 * 4
    assert n1 >= delta + 4 * 256 * 256 * 4        # delta rows + fp32 accumulator over (1, H, S, T)
    assert n0 >= delta + 2 * 4 * 256 * 128 * 4    # without dbias: delta rows + the one-kernel backward's fp32 dq sums


def test_jax_ffi_layer_is_complete_and_consistent():
    """The JAX binding cannot run here (no jax, no XLA FFI headers); it must at least compile as Python, import
    without jax, and agree with the C++ shim on the handler symbols and attribute names, and the shim must use
    only entry points the header declares."""
    import py_compile

    py_compile.compile(str(ROOT / "nitrix_b200" / "jax_ffi.py"), doraise=True)
    from nitrix_b200 import jax_ffi

    shim = (ROOT / "ffi" / "nb200_ffi.cc").read_text()
    symbols = set(re.findall(r"XLA_FFI_DEFINE_HANDLER_SYMBOL\(\s*(\w+)", shim))
    assert symbols == {jax_ffi.FWD_SYMBOL, jax_ffi.BWD_SYMBOL}
    fwd_block, bwd_block = shim.split("XLA_FFI_DEFINE_HANDLER_SYMBOL(")[1:3]
    assert tuple(re.findall(r'\.Attr<\w+>\("(\w+)"\)', fwd_block)) == jax_ffi.FWD_ATTRS
    assert tuple(re.findall(r'\.Attr<\w+>\("(\w+)"\)', bwd_block)) == jax_ffi.BWD_ATTRS
    assert fwd_block.count(".Arg<") == 5 and fwd_block.count(".Ret<") == 3
    assert bwd_block.count(".Arg<") == 8 and bwd_block.count(".Ret<") == 5
    header = (ROOT / "include" / "nitrix_b200_attention.h").read_text()
    for called in set(re.findall(r"\b(nb200_\w+)\s*\(", shim)) - symbols:
        assert re.search(rf"NB200_API[^;]*\b{called}\s*\(", header), called
    # the trace-time queries go through the C ABI without a GPU: a covered problem gives a size, a declined one raises
    key = ((2, 4, 256, 64), (2, 4, 256, 64), (2, 4, 256, 64), "bfloat16", None, None, (2, 1, 256, 256), 0.125, False, False)
    assert jax_ffi._workspace_bytes(0, *key) >= 2 * 256 * 8 * 4
    with pytest.raises(jax_ffi.NotCovered):
        jax_ffi._workspace_bytes(0, (1, 2, 8, 512), (1, 2, 8, 512), (1, 2, 8, 512), "float32", None, None, None, 0.1, False, False)
    with pytest.raises(ImportError):
        jax_ffi.register()


def test_jax_norm_ffi_layer_is_complete_and_consistent():
    """The LayerNorm FFI shim and its JAX module: the module compiles and imports without jax, and its handler
    symbols and attribute lists are the ones the C++ file binds (neither can run here: no jax, no XLA headers)."""
    import py_compile

    py_compile.compile(str(ROOT / "nitrix_b200" / "jax_norm_ffi.py"), doraise=True)
    from nitrix_b200 import jax_norm_ffi as J

    shim = (ROOT / "ffi" / "nb200_norm_ffi.cc").read_text()
    symbols = set(re.findall(r"XLA_FFI_DEFINE_HANDLER_SYMBOL\((\w+),", shim))
    assert symbols == {J.FWD_SYMBOL, J.BWD_SYMBOL}
    fwd_block, bwd_block = shim.split("XLA_FFI_DEFINE_HANDLER_SYMBOL(")[1:3]
    assert tuple(re.findall(r'\.Attr<\w+>\("(\w+)"\)', fwd_block)) == J.FWD_ATTRS
    assert tuple(re.findall(r'\.Attr<\w+>\("(\w+)"\)', bwd_block)) == J.BWD_ATTRS
    # every entry point the shim calls is declared in the header
    header = (ROOT / "include" / "nitrix_b200_norm.h").read_text()
    for name in set(re.findall(r"\b(nb200_layer_norm_\w+)\(", shim)) - symbols:
        assert name in header, name
    # the trace-time workspace query goes through the real library
    assert J.workspace_bytes(8192, 2048, "bfloat16") >= 2 * 2048 * 4


def test_jax_scan_ffi_layer_is_complete_and_consistent():
    """The selective-scan FFI shim and its JAX module: the module compiles and imports without jax, and its handler
    symbols and attribute lists are the ones the C++ file binds (neither can run here: no jax, no XLA headers)."""
    import py_compile

    py_compile.compile(str(ROOT / "nitrix_b200" / "jax_scan_ffi.py"), doraise=True)
    from nitrix_b200 import jax_scan_ffi as J

    shim = (ROOT / "ffi" / "nb200_scan_ffi.cc").read_text()
    symbols = set(re.findall(r"XLA_FFI_DEFINE_HANDLER_SYMBOL\((\w+),", shim))
    assert symbols == {J.FWD_SYMBOL, J.BWD_SYMBOL}
    fwd_block, bwd_block = shim.split("XLA_FFI_DEFINE_HANDLER_SYMBOL(")[1:3]
    assert tuple(re.findall(r'\.Attr<\w+>\("(\w+)"\)', fwd_block)) == J.FWD_ATTRS
    assert tuple(re.findall(r'\.Attr<\w+>\("(\w+)"\)', bwd_block)) == J.BWD_ATTRS
    header = (ROOT / "include" / "nitrix_b200_scan.h").read_text()
    for name in set(re.findall(r"\b(nb200_selective_scan_\w+)\(", shim)) - symbols:
        assert name in header, name
    ck, ws = J.scratch_bytes(8, 1024, 2048, 16, "bfloat16")
    assert ck == 8 * 128 * 2048 * 16 * 4 and ws >= 2 * 8 * 1024 * 16 * 4
