"""Host-side behaviour of the public functions that needs no GPU: argument validation with the
reference's error texts, refusal to run anywhere but on a B200, fake-tensor shape inference."""

import pytest
import torch

import triton_sigmoid_b200 as m
from triton_sigmoid_b200 import ops


def _qkv(B=2, T=32, H=2, D=64, dtype=torch.float16):
    return [torch.zeros(B, T, H, D, dtype=dtype) for _ in range(3)]


def test_exports_match_reference_package():
    """The reference's three names, plus what it does not have: the packed variable-length entry point and
    the two run-time helpers (accurate-sigmoid switch, device health word)."""
    assert set(m.__all__) == {"sigmoid_attention", "sigmoid_attention_padded", "sigmoid_attention_ref",
                              "sigmoid_attention_varlen", "accurate_sigmoid", "device_status"}


def test_accurate_switch_follows_the_reference_variable(monkeypatch):
    """TRITON_SIGMOID_ACCURATE takes the reference's values (kernel_utils.py:190-193 there), read per call;
    the context manager overrides it."""
    monkeypatch.delenv("TRITON_SIGMOID_ACCURATE", raising=False)
    assert not ops._accurate()
    for v in ("1", "true", "YES", "On"):
        monkeypatch.setenv("TRITON_SIGMOID_ACCURATE", v)
        assert ops._accurate()
    monkeypatch.setenv("TRITON_SIGMOID_ACCURATE", "0")
    assert not ops._accurate()
    with m.accurate_sigmoid(True):
        assert ops._accurate() and ops._flags(True) == 3
        with m.accurate_sigmoid(False):
            assert not ops._accurate() and ops._flags(False) == 0
        assert ops._accurate()
    assert not ops._accurate()


def test_varlen_argument_errors():
    q = torch.zeros(10, 2, 64, dtype=torch.float16)
    cu = torch.tensor([0, 4, 10], dtype=torch.int32)
    with pytest.raises(ValueError, match="3D tensors"):
        m.sigmoid_attention_varlen(q[None], q[None], q[None], cu, cu, 6, 6)
    with pytest.raises(ValueError, match="Key and value shapes must match"):
        m.sigmoid_attention_varlen(q, q, q[:5], cu, cu, 6, 6)
    with pytest.raises(ValueError, match="Number of heads mismatch"):
        m.sigmoid_attention_varlen(q, q[:, :1], q[:, :1], cu, cu, 6, 6)
    with pytest.raises(ValueError, match="cu_seqlens_q and cu_seqlens_k"):
        m.sigmoid_attention_varlen(q, q, q, cu, cu[:2], 6, 6)
    with pytest.raises(ValueError, match="score_mod must have shape"):
        m.sigmoid_attention_varlen(q, q, q, cu, cu, 6, 6, score_mod=torch.zeros(3))
    with pytest.raises(NotImplementedError, match="float64"):
        m.sigmoid_attention_varlen(q.double(), q.double(), q.double(), cu, cu, 6, 6)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        m.sigmoid_attention_varlen(q, q, q, cu, cu, 6, 6)


@pytest.mark.parametrize("fn", [m.sigmoid_attention, m.sigmoid_attention_padded])
def test_shape_errors(fn):
    q, k, v = _qkv()
    with pytest.raises(ValueError, match="Expected query, key, and value to be 4D tensors"):
        fn(q[0], k, v)
    with pytest.raises(ValueError, match="Batch size mismatch"):
        fn(q, k[:1], v)
    with pytest.raises(ValueError, match="Number of heads mismatch"):
        fn(q, k, v[:, :, :1])
    with pytest.raises(ValueError, match="Head dimension mismatch"):
        fn(q, k[..., :32], v)


def test_dense_requires_equal_lengths():
    q, k, v = _qkv()
    with pytest.raises(ValueError, match="Dense attention requires same sequence length"):
        m.sigmoid_attention(q, k[:, :16], v[:, :16])


def test_padded_requires_matching_kv():
    q, k, v = _qkv()
    with pytest.raises(ValueError, match="Key and value sequence lengths must match"):
        m.sigmoid_attention_padded(q, k, v[:, :16])


@pytest.mark.parametrize("fn", [m.sigmoid_attention, m.sigmoid_attention_padded])
def test_score_mod_shape(fn):
    q, k, v = _qkv()
    with pytest.raises(ValueError, match="score_mod must have shape"):
        fn(q, k, v, score_mod=torch.zeros(2, 31))


def test_seq_lens_shape():
    q, k, v = _qkv()
    with pytest.raises(ValueError, match="seq_lens_k must have shape"):
        m.sigmoid_attention_padded(q, k, v, seq_lens_k=torch.zeros(3, dtype=torch.int32))
    with pytest.raises(ValueError, match="seq_lens_q must have shape"):
        m.sigmoid_attention_padded(q, k, v, seq_lens_q=torch.zeros(2, 1, dtype=torch.int32))


def test_float32_is_accepted_and_other_dtypes_are_refused():
    """float32 is a supported dtype (exact kernels), so on CPU tensors it gets as far as the
    device check; float64 is refused outright, never downcast."""
    q, k, v = _qkv(dtype=torch.float32)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        m.sigmoid_attention(q, k, v)
    q, k, v = _qkv(dtype=torch.float64)
    with pytest.raises(NotImplementedError, match="float64"):
        m.sigmoid_attention(q, k, v)


def test_no_cpu_fallback():
    q, k, v = _qkv()
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        m.sigmoid_attention(q, k, v)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        m.sigmoid_attention_padded(q, k, v)


def test_ops_are_registered_with_reference_names():
    ns = torch.ops.sigattn_b200
    for name in ("sigmoid_attention_fwd", "sigmoid_attention_bwd", "sigmoid_attn_padded_fwd", "sigmoid_attn_padded_bwd"):
        assert hasattr(ns, name)
    schema = str(ops.sigmoid_attention_fwd_op._opoverload._schema)
    assert "Tensor? score_mod" in schema and "bool is_causal" in schema


def test_fake_kernels_infer_shapes():
    from torch._subclasses.fake_tensor import FakeTensorMode

    with FakeTensorMode():
        q = torch.empty(3, 40, 2, 64, dtype=torch.bfloat16)
        k = torch.empty(3, 72, 2, 64, dtype=torch.bfloat16)
        bias = torch.empty(3)
        lens = torch.empty(3, dtype=torch.int32)
        o = ops.sigmoid_attn_padded_fwd_op(q, k, k, lens, lens, bias, None, 0.125, False)
        assert o.shape == q.shape and o.dtype == q.dtype
        dq, dk, dv = ops.sigmoid_attn_padded_bwd_op(q, k, k, o, lens, lens, bias, None, 0.125, True)
        assert dq.shape == q.shape and dk.shape == k.shape and dv.shape == k.shape
        o2 = ops.sigmoid_attention_fwd_op(q, q, q, bias, None, 0.125, True)
        assert o2.shape == q.shape


def test_torch_reference_matches_oracle():
    from oracle import sigattn_oracle as orc

    torch.manual_seed(3)
    q, k, v = [torch.randn(2, 48, 2, 16) for _ in range(3)]
    lens = torch.tensor([48, 17], dtype=torch.int32)
    a = m.sigmoid_attention_ref(q, k, v, seq_lens_k=lens, seq_lens_q=lens, causal=True)
    b = orc.sigattn_forward(q, k, v, seq_lens_k=lens, seq_lens_q=lens, is_causal=True)
    assert (a - b).abs().max() < 2e-5
