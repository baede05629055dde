"""HuggingFace integration end to end: a small random-init Llama with
``attn_implementation = "attnfuse"`` against the same weights on SDPA -- prefill logits, a
training step's gradients, and a cached decode step."""
import pytest
import torch

transformers = pytest.importorskip("transformers")

pytestmark = pytest.mark.gpu
DEV = "cuda"


def tiny_llama(dtype):
    import attentionfuse_b200.integrations.hf  # noqa: F401  (registers the backend)
    cfg = transformers.LlamaConfig(vocab_size=128, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                                   num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                                   max_position_embeddings=1024, attn_implementation="sdpa")
    torch.manual_seed(0)
    model = transformers.LlamaForCausalLM(cfg).to(device=DEV, dtype=dtype)
    return model


def use_backend(model, name):
    if hasattr(model, "set_attn_implementation"):
        try:
            model.set_attn_implementation(name)
            return
        except Exception:
            pass
    model.config._attn_implementation = name


def test_registration_on_import():
    import attentionfuse_b200.integrations.hf as hf
    from transformers.modeling_utils import ALL_ATTENTION_FUNCTIONS
    assert ALL_ATTENTION_FUNCTIONS["attnfuse"] is hf.attnfuse_attention_forward
    import attnfuse.integrations.hf as alias          # the reference's import path
    assert alias.attnfuse_attention_forward is hf.attnfuse_attention_forward


def test_prefill_logits_match_sdpa():
    model = tiny_llama(torch.bfloat16).eval()
    ids = torch.randint(0, 128, (2, 300), device=DEV)
    with torch.no_grad():
        use_backend(model, "sdpa")
        want = model(ids).logits.float()
        use_backend(model, "attnfuse")
        from attentionfuse_b200.runtime import _lib
        before = _lib.launch_count()
        got = model(ids).logits.float()
        assert _lib.launch_count() - before >= 2, "the attnfuse backend did not launch this library's kernels"
    err = (got - want).abs().max().item()
    assert err < 6e-2 and (got - want).norm() / want.norm() < 2e-2, err


def test_training_step_gradients_match_sdpa():
    model = tiny_llama(torch.bfloat16).train()
    ids = torch.randint(0, 128, (2, 200), device=DEV)
    grads = {}
    for name in ("sdpa", "attnfuse"):
        use_backend(model, name)
        model.zero_grad(set_to_none=True)
        out = model(ids, labels=ids)
        out.loss.backward()
        grads[name] = (out.loss.item(), model.model.layers[0].self_attn.q_proj.weight.grad.float().clone(),
                       model.model.layers[1].self_attn.v_proj.weight.grad.float().clone())
    assert abs(grads["sdpa"][0] - grads["attnfuse"][0]) < 2e-2
    for a, b in zip(grads["sdpa"][1:], grads["attnfuse"][1:]):
        assert (a - b).norm() / a.norm() < 5e-2


def test_cached_decode_step_matches_sdpa():
    model = tiny_llama(torch.float16).eval()
    ids = torch.randint(0, 128, (2, 400), device=DEV)
    outs = {}
    with torch.no_grad():
        for name in ("sdpa", "attnfuse"):
            use_backend(model, name)
            pre = model(ids[:, :-1], use_cache=True)
            step = model(ids[:, -1:], past_key_values=pre.past_key_values, use_cache=True)
            outs[name] = step.logits.float()
    assert (outs["sdpa"] - outs["attnfuse"]).abs().max().item() < 3e-2


def test_chunked_prefill_against_cache_stays_on_the_kernel(monkeypatch):
    """A chunk of queries at the end of a longer cache, with HF's additive causal mask: served by
    the kernel with a position offset, not by the SDPA fall-back."""
    import attentionfuse_b200.integrations.hf as hf
    from transformers.modeling_utils import ALL_ATTENTION_FUNCTIONS
    from oracle import attention_oracle as orc
    from tests._util import assert_close, qkv
    B, Hq, Hkv, N_q, N_kv, D = 2, 4, 2, 100, 300, 64
    Q, K, V = qkv(4100, B, Hq, Hkv, N_q, N_kv, D, torch.bfloat16)
    off = N_kv - N_q
    i = torch.arange(N_q).view(N_q, 1) + off
    j = torch.arange(N_kv).view(1, N_kv)
    mask = torch.zeros(B, 1, N_q, N_kv, dtype=torch.bfloat16)
    mask.masked_fill_((j > i).view(1, 1, N_q, N_kv), torch.finfo(torch.bfloat16).min)

    def no_fallback(*a, **k):
        raise AssertionError("fell back to SDPA")
    monkeypatch.setitem(ALL_ATTENTION_FUNCTIONS, "sdpa", no_fallback)
    out, _ = hf.attnfuse_attention_forward(torch.nn.Identity(), Q.to(DEV), K.to(DEV), V.to(DEV), mask.to(DEV),
                                           is_causal=False)
    want = orc.attention(Q, K, V, causal=True, q_offset=off)
    assert_close(out.transpose(1, 2), want, torch.bfloat16, what="HF chunked prefill")
