"""The C-ABI library loads, exports what include/sigattn_b200.h declares, and rejects bad
arguments before touching a GPU.  No compute happens here."""

import ctypes
import os
import re

import pytest

from tests.conftest import ROOT
from triton_sigmoid_b200 import _cabi
from triton_sigmoid_b200.build import LIB_PATH, build


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(LIB_PATH):
        build()
    return _cabi.load()


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "sigattn_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sigattn_[a-z_0-9]+)\s*\(", text)))


def test_header_and_binding_agree():
    assert _declared_functions() == sorted(_cabi.EXPORTED_SYMBOLS)


def test_every_declared_symbol_is_exported(lib):
    for name in _declared_functions():
        assert getattr(lib, name) is not None


def test_query(lib):
    assert lib.sigattn_query(_cabi.Q_ABI_VERSION) == 2
    assert lib.sigattn_query(_cabi.Q_SM_ARCH) == 100
    assert lib.sigattn_query(_cabi.Q_MAX_HEAD_DIM) == 128
    assert lib.sigattn_query(_cabi.Q_PARAMS_SIZE) == ctypes.sizeof(_cabi.SigAttnParams)
    assert lib.sigattn_query(12345) == -1


def test_workspace_bytes(lib):
    assert lib.sigattn_bwd_workspace_bytes(2, 100, 3, 64) == 2 * 100 * 3 * 64 * 4
    assert lib.sigattn_bwd_workspace_bytes(0, 100, 3, 64) == 0


def _params(**kw):
    p = _cabi.SigAttnParams()
    p.struct_bytes = ctypes.sizeof(_cabi.SigAttnParams)
    p.dtype, p.B, p.H, p.D, p.Tq, p.Tk = 0, 1, 1, 64, 128, 128
    p.q = p.k = p.v = p.o = 0x1000
    for k, v in kw.items():
        setattr(p, k, v)
    return p


def test_null_params_rejected(lib):
    assert lib.sigattn_fwd(None) < 0
    assert b"NULL" in lib.sigattn_last_error()


@pytest.mark.parametrize("kw,needle", [
    (dict(struct_bytes=8), b"ABI mismatch"),
    (dict(dtype=7), b"unsupported dtype"),
    (dict(D=48), b"unsupported head dimension"),
    (dict(B=-1), b"negative extent"),
    (dict(H=70000), b"65535"),
    (dict(q=None), b"must not be NULL"),
    (dict(o=None), b"o must not be NULL"),
    (dict(cu_seqlens_q=0x2000), b"needs both cu_seqlens_q and cu_seqlens_k"),
    (dict(cu_seqlens_q=0x2000, cu_seqlens_k=0x2000, seq_lens_k=0x3000), b"seq_lens_q / seq_lens_k must be NULL"),
    (dict(cu_seqlens_q=0x2000, cu_seqlens_k=0x2000, total_q=-1), b"negative total_q"),
])
def test_bad_arguments_rejected_before_any_cuda_call(lib, kw, needle):
    rc = lib.sigattn_fwd(ctypes.byref(_params(**kw)))
    assert rc < 0
    assert needle in lib.sigattn_last_error()


def test_backward_needs_gradient_pointers(lib):
    rc = lib.sigattn_bwd(ctypes.byref(_params()))
    assert rc < 0 and b"dout, dq, dk, dv" in lib.sigattn_last_error()


def test_empty_batch_is_a_no_op(lib):
    assert lib.sigattn_fwd(ctypes.byref(_params(B=0))) == 0
    assert lib.sigattn_last_error() == b""


def test_documented_reference_side_binding_is_runnable_python():
    """The ctypes stub shown to the reference's maintainers imports and defines its op body
    with the names this package really exports (executed up to, not including, a call)."""
    import os
    import re

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    text = open(os.path.join(root, "INTEGRATION.md")).read()
    block = re.search(r"```python\n(.*?)```", text, re.S).group(1)
    ns = {}
    exec(compile(block, "INTEGRATION.md", "exec"), ns)
    assert callable(ns["sigmoid_attention_fwd_op"]) and isinstance(ns["USE_ACCURATE_SIGMOID"], bool)
