"""Seeded synthetic stand-ins for the reference's checkpoints and calibration sets.

The reference calibrates real checkpoints on WikiText-2 / PTB / C4 samples
(run.py:19-71, datautils.py:306-341); neither is available offline.  These
builders create random-init models of the same shapes and uniform token-id
calibration batches of the same sizes (128 sequences x 2048 tokens).
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch

# name -> (architecture, config kwargs).  Shapes follow the public model cards.
MODEL_SHAPES = {
    "opt-tiny": ("opt", dict(hidden_size=256, ffn_dim=1024, num_hidden_layers=2, num_attention_heads=4,
                             vocab_size=2048, max_position_embeddings=2048, dtype=torch.float16)),
    "opt-1.3b": ("opt", dict(hidden_size=2048, ffn_dim=8192, num_hidden_layers=24, num_attention_heads=32,
                             vocab_size=50272, max_position_embeddings=2048, dtype=torch.float16)),
    "opt-6.7b": ("opt", dict(hidden_size=4096, ffn_dim=16384, num_hidden_layers=32, num_attention_heads=32,
                             vocab_size=50272, max_position_embeddings=2048, dtype=torch.float16)),
    "opt-66b": ("opt", dict(hidden_size=9216, ffn_dim=36864, num_hidden_layers=64, num_attention_heads=72,
                            vocab_size=50272, max_position_embeddings=2048, dtype=torch.float16)),
    "llama-3-8b": ("llama", dict(hidden_size=4096, intermediate_size=14336, num_hidden_layers=32,
                                 num_attention_heads=32, num_key_value_heads=8, vocab_size=128256,
                                 max_position_embeddings=8192, dtype=torch.bfloat16)),
    "llama-tiny": ("llama", dict(hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                                 num_attention_heads=4, num_key_value_heads=2, vocab_size=2048,
                                 max_position_embeddings=2048, dtype=torch.bfloat16)),
}


def resolve_shape(model_name: str) -> Optional[str]:
    """Maps names like `facebook/opt-6.7b` or `synthetic:opt-6.7b` onto a key of MODEL_SHAPES."""
    key = model_name.lower().split("/")[-1].replace("synthetic:", "").replace("meta-llama-", "llama-")
    return key if key in MODEL_SHAPES else None


def build_synthetic_model(model_name: str, n_layers: Optional[int] = None, seed: int = 0,
                          fill_device: Optional[str] = None, attn: str = "sdpa"):
    """Random-init model of the named shape: weights ~ N(0, 0.02^2), LayerNorm weight 1, biases 0.

    Parameters live on the CPU (pinned when CUDA is present) as in the reference's
    layer-streaming flow (run.py:238, :381); the values are drawn on `fill_device`
    when given, which is much faster than CPU sampling for billions of weights.
    """
    key = resolve_shape(model_name)
    if key is None:
        raise ValueError(f"no synthetic shape for {model_name!r}; known: {sorted(MODEL_SHAPES)}")
    arch, kw = MODEL_SHAPES[key]
    kw = dict(kw)
    dtype = kw.pop("dtype")
    if n_layers is not None:
        kw["num_hidden_layers"] = n_layers
    if arch == "opt":
        from transformers import OPTConfig, OPTForCausalLM
        cfg = OPTConfig(word_embed_proj_dim=kw["hidden_size"], **kw)
        cls = OPTForCausalLM
    else:
        from transformers import LlamaConfig, LlamaForCausalLM
        cfg = LlamaConfig(**kw)
        cls = LlamaForCausalLM
    cfg._attn_implementation = attn
    cfg.use_cache = False
    with torch.device("meta"):
        model = cls(cfg)
    model = model.to(dtype).to_empty(device="cpu")
    gen_dev = fill_device or "cpu"
    g = torch.Generator(device=gen_dev).manual_seed(seed)
    pin = torch.cuda.is_available()
    for name, p in model.named_parameters():
        if p.dim() >= 2:
            vals = (torch.randn(p.shape, generator=g, device=gen_dev, dtype=torch.float32) * 0.02).to(dtype)
        elif name.endswith("weight"):
            vals = torch.ones(p.shape, dtype=dtype, device=gen_dev)      # norm gains
        else:
            vals = torch.zeros(p.shape, dtype=dtype, device=gen_dev)     # biases
        host = torch.empty(p.shape, dtype=dtype, pin_memory=pin)
        host.copy_(vals)
        p.data = host
    _reinit_buffers(model)
    model.seqlen = min(cfg.max_position_embeddings, 2048)
    model.eval()
    model.crb_model_name = f"synthetic/{key}"
    return model


def _reinit_buffers(model):
    """Buffers created under the meta device (rotary inv_freq) hold no values after to_empty:
    recompute them in float32 with the module's own initialiser."""
    for mod in model.modules():
        if not (hasattr(mod, "inv_freq") and hasattr(mod, "config")):
            continue
        rope_type = getattr(mod, "rope_type", "default")
        if rope_type == "default" and hasattr(mod, "compute_default_rope_parameters"):
            init = mod.compute_default_rope_parameters
        else:
            from transformers.modeling_rope_utils import ROPE_INIT_FUNCTIONS
            init = ROPE_INIT_FUNCTIONS[rope_type]
        inv_freq, scaling = init(mod.config, "cpu")
        mod.register_buffer("inv_freq", inv_freq.float(), persistent=False)
        if hasattr(mod, "original_inv_freq"):
            mod.register_buffer("original_inv_freq", inv_freq.float().clone(), persistent=False)
        mod.attention_scaling = scaling


def synthetic_calibration(vocab_size: int, nsamples: int = 128, seqlen: int = 2048,
                          seed: int = 0) -> List[Tuple[torch.Tensor, None]]:
    """`nsamples` batches of one sequence of uniform token ids, like get_loaders' train list."""
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, vocab_size, (nsamples, seqlen), generator=g)
    return [(ids[j:j + 1], None) for j in range(nsamples)]


def single_linear_case(R: int = 2048, C: int = 2048, nseq: int = 128, seqlen: int = 2048,
                       seed: int = 1, device: str = "cpu"):
    """The single-linear configuration: W ~ N(0, 0.02^2); X ~ N(0, 1) with 1 % of the channels x20.

    Returns (W, channel list, generator of per-sequence X blocks) with the seeds used
    by tests/golden/make_golden.py, so that the golden outputs apply.
    """
    g = torch.Generator().manual_seed(seed)
    W = torch.randn(R, C, generator=g) * 0.02
    ch = torch.randperm(C, generator=g)[: C // 100]

    def sequences():
        for j in range(nseq):
            gx = torch.Generator().manual_seed(1000 + j)
            x = torch.randn(seqlen, C, generator=gx)
            x[:, ch] *= 20
            yield x.to(device)

    return W, ch, sequences
