"""Mamba-2 / short-convolution / hybrid stacks on the GPU path (bf16 GEMM kernels + attention kernels) against the same
weights evaluated in fp32 on the CPU."""
import pytest
import torch

from primus_b200.ops import _lib

pytestmark = pytest.mark.gpu


def _pair(**kw):
    from primus_b200.models.config import TransformerConfig
    from primus_b200.models.gpt import GPTModel
    from primus_b200.parallel import state as ps

    ps.destroy_model_parallel()
    ps.initialize_model_parallel()
    base = dict(hidden_size=256, ffn_hidden_size=512, num_attention_heads=2, num_query_groups=2, kv_channels=128,
                vocab_size=1024, seq_length=256, untie_embeddings_and_output_weights=False)
    base.update(kw)
    torch.manual_seed(0)
    gpu = GPTModel(TransformerConfig(**dict(base, params_dtype="bf16")), "cuda")
    cpu = GPTModel(TransformerConfig(**dict(base, params_dtype="fp32")), "cpu")
    cpu.load_state_dict({k: v.detach().float().cpu() for k, v in gpu.state_dict().items()})
    return gpu, cpu


@pytest.mark.parametrize("kw", [
    dict(num_layers=4, model_type="mamba", is_hybrid_model=True, hybrid_override_pattern="M-*-", mamba_head_dim=64,
         mamba_num_groups=2, mamba_state_dim=32, mamba_chunk_size=64),
    dict(num_layers=3, lfm_layer_types=["conv", "full_attention", "conv"], qk_layernorm=True),
    dict(num_layers=4, model_type="mamba", is_hybrid_model=True, linear_attention_type="gdn", hybrid_override_pattern="M-*-",
         linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=64, linear_value_head_dim=64),
], ids=["mamba_hybrid", "lfm2", "gated_delta_net"])
def test_mixer_stacks_match_fp32_cpu(kw):
    gpu, cpu = _pair(**kw)
    tokens = torch.randint(0, 1024, (2, 256))
    labels = torch.randint(0, 1024, (2, 256))
    with torch.no_grad():
        ref = cpu(tokens, labels).float()
    loss = gpu(tokens.cuda(), labels.cuda())
    loss.float().mean().backward()
    torch.cuda.synchronize()
    _lib.check_status()
    got = loss.detach().float().cpu()
    assert (got - ref).abs().max() <= 0.05 * ref.abs().max(), ((got - ref).abs().max(), ref.abs().max())
    assert abs(got.mean() - ref.mean()) <= 5e-3 * ref.mean()
    grads = [p.grad if p.grad is not None else getattr(p, "main_grad", None) for p in gpu.parameters()]
    assert all(g is not None and torch.isfinite(g.float()).all() for g in grads)
