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
