"""Named config.json dictionaries for the random-weights mode.  They are data handed to the
configuration class like any model folder's config.json; nothing in the engine reads them.

``tiny`` has the sizes of the reference's ``ModelConfig.tiny()`` (src/llmserve/config.py:26-37);
``tinyllama-1.1b`` those of its defaults (src/llmserve/config.py:10-20).
"""

from __future__ import annotations


def _llama(**kw) -> dict:
    base = {
        "architectures": ["LlamaForCausalLM"],
        "model_type": "llama",
        "hidden_act": "silu",
        "rope_theta": 10000.0,
        "rms_norm_eps": 1e-5,
        "tie_word_embeddings": False,
    }
    base.update(kw)
    return base


def _nurolorn(width: int, ff: int, heads: int, rank: int, rot: int, window: int, pattern: str, loop, vocab: int = 32000) -> dict:
    """``pattern``: one letter a layer, L latent attention, G minGRU, W window attention; every layer has a dense feed-forward."""
    head = 64
    kinds = {
        "L": lambda: {"type": "latent_attention", "mixer": {"heads": heads, "dim": head, "rot_dim": rot, "vdim": head, "kv_rank": rank,
                                                            "scale": (head + rot) ** -0.5, "rot": {"base": 10000.0, "dims": rot}}},
        "G": lambda: {"type": "mingru", "mixer": {"width": width}},
        "W": lambda: {"type": "attention", "mixer": {"heads": heads, "kv_heads": max(1, heads // 8), "dim": head, "vdim": head,
                                                     "scale": head ** -0.5, "mask": {"size": window}}},
    }
    layers = [{**kinds[c](), "mlp": {"kind": "dense", "ff": ff}} for c in pattern]
    return {
        "architecture": "Nurolorn", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": 1e-6, "groups": 2},
        "residual_mult": 0.7, "logit_scale": 1.0, "loop": dict(zip(("start", "stop", "times"), loop)),
    }


def _kafepel(width: int, layers: int, heads: int, kv_heads: int, ff: int, experts: int, top: int, expert_ff: int, shared_ff: int,
             vocab: int = 32000) -> dict:
    """Layers alternate between a dense and a routed feed-forward; the attention branch has heads of 64 lanes, the
    retention branch half as many heads with keys of 64 and values of 128 lanes (decays ``1 - 2^-(5 + h/2)``)."""
    head = 64
    left = {"heads": heads, "kv_heads": kv_heads, "dim": head, "vdim": head, "scale": head ** -0.5, "softcap": 30.0,
            "rot": {"base": 500000.0, "dims": head, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}
    r_heads = heads // 2
    right = {"heads": r_heads, "dim": head, "vdim": 2 * head, "decay": [1.0 - 2.0 ** -(5.0 + h / 2.0) for h in range(r_heads)],
             "rot": {"base": 10000.0, "dims": head}}
    dense = {"kind": "dense", "ff": ff}
    moe = {"kind": "moe", "router": {"experts": experts, "top": top, "scale": 2.5}, "expert": {"ff": expert_ff}, "shared": {"ff": shared_ff}}
    return {
        "architecture": "Kafepel", "vocab": vocab, "width": width, "embedding": {"scale": float(width) ** 0.5}, "norm": {"eps": 1e-6},
        "layers": [{"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": dense if i % 2 == 0 else moe} for i in range(layers)],
    }


def _nudodra(width: int, pattern: str, heads: int, kv_heads: int, experts: int, top: int, expert_ff: int, shared_ff: int, streams: int = 4,
             vocab: int = 32000) -> dict:
    """``pattern``: one letter a layer, P side-by-side mixers, A attention with keys and values of its own, a attention that
    reads the pages of the last A in front of it.  Heads of 64 lanes; the recurrent branch has half as many heads with keys
    of 64 and values of 128 lanes and a decay product of inner size 64; every layer has the table-routed feed-forward."""
    head = 64
    left = {"heads": heads, "kv_heads": kv_heads, "dim": head, "vdim": head, "scale": head ** -0.5, "rot": {"base": 10000.0, "dims": head // 2}}
    right = {"heads": heads // 2, "dim": head, "vdim": 2 * head, "tau": 8.0, "rank": 64}
    attention = {"heads": heads, "kv_heads": kv_heads, "dim": head, "vdim": head, "scale": head ** -0.5, "q_temp": {"coef": 0.1, "every": 1024}}
    moe = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": expert_ff, "limit": 7.0}, "shared": {"ff": shared_ff, "limit": 7.0}}
    layers, last = [], None
    for i, c in enumerate(pattern):
        if c == "P":
            layers.append({"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": 0.7, "right_scale": 0.7}, "mlp": moe})
        else:
            mixer = dict(attention) if c == "A" else {**attention, "kv_from": last}
            last = i if c == "A" else last
            layers.append({"type": "attention", "mixer": mixer, "mlp": moe})
    return {"architecture": "Nudodra", "vocab": vocab, "width": width, "streams": streams, "norm": {"eps": 1e-6}, "layers": layers}


def _tenotar(width: int, pattern: str, heads: int, kv_heads: int, rank: int, q_rank: int, dense_ff: int, experts: int, top: int, expert_ff: int,
             shared_ff: int, span: int = 512, vocab: int = 32000) -> dict:
    """``pattern``: one letter a layer, W attention with a window that keeps the first tokens, C attention behind a short
    convolution over blocks of positions, L attention through latents.  Heads of 64 lanes, a rotated part of 32; windows and
    blocks of ``span`` positions; the first layer's feed-forward is dense, the others' a mixture of gated experts."""
    head = 64
    kinds = {
        "W": lambda: {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": head, "vdim": head, "scale": head ** -0.5,
                                                     "mask": {"size": span, "keep_first": 16}, "rot": {"base": 10000.0, "dims": head}, "v_mix": True}},
        "C": lambda: {"type": "attention_2", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": head, "vdim": head, "scale": head ** -0.5,
                                                       "mask": {"size": span}, "conv": 4, "softcap": 30.0, "v_mix": True}},
        "L": lambda: {"type": "latent_attention", "mixer": {"heads": heads, "dim": head, "rot_dim": 32, "vdim": head, "kv_rank": rank, "q_rank": q_rank,
                                                            "scale": (head + 32) ** -0.5, "mask": {"size": span}, "rot": {"base": 10000.0, "dims": 32}}},
    }
    moe = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": expert_ff}, "shared": {"ff": shared_ff}}
    layers = [{**kinds[c](), "mlp": {"kind": "dense", "ff": dense_ff} if i == 0 else moe} for i, c in enumerate(pattern)]
    return {"architecture": "Tenotar", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": 1e-6}, "logit_scale": 1.0}


PRESETS: dict[str, dict] = {
    # Tenotar at the sizes of the Nudodra and Kafepel presets below (the design has no published sizes)
    "tenotar-small": _tenotar(1024, "WCLWCLWC", 16, 4, 128, 384, 2816, 16, 2, 512, 1024),
    "tenotar-1b": _tenotar(2048, "WCLWCLWCLWCL", 32, 8, 256, 768, 5632, 32, 4, 704, 1408),
    # Nudodra at the sizes of the Kafepel presets below (the design has no published sizes)
    "nudodra-small": _nudodra(1024, "PAaPAaPP", 16, 4, 16, 2, 512, 1024),
    "nudodra-1b": _nudodra(2048, "PAaPAaPAaPPA", 32, 8, 32, 4, 704, 1408),
    # Kafepel at sizes that resemble real layers (the design has no published sizes)
    "kafepel-small": _kafepel(1024, 8, 16, 4, 2816, 16, 2, 512, 1024),
    "kafepel-1b": _kafepel(2048, 12, 32, 8, 5632, 32, 4, 704, 1408),
    # Nurolorn at sizes that resemble real layers (the design has no published sizes): a stretch of four layers runs twice
    "nurolorn-small": _nurolorn(1024, 4096, 16, 128, 32, 512, "LLGWLL", (1, 5, 2)),
    "nurolorn-1b": _nurolorn(2048, 8192, 32, 256, 32, 1024, "LLGWLLGWLL", (2, 8, 2)),
    "tiny": _llama(
        vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
        num_key_value_heads=2, max_position_embeddings=512,
    ),
    "tinyllama-1.1b": _llama(
        vocab_size=32000, hidden_size=2048, intermediate_size=5632, num_hidden_layers=22, num_attention_heads=32,
        num_key_value_heads=4, max_position_embeddings=2048,
    ),
    "llama2-7b": _llama(
        vocab_size=32000, hidden_size=4096, intermediate_size=11008, num_hidden_layers=32, num_attention_heads=32,
        num_key_value_heads=32, max_position_embeddings=4096,
    ),
    "llama3-8b": _llama(
        vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32, num_attention_heads=32,
        num_key_value_heads=8, max_position_embeddings=8192, rope_theta=500000.0,
    ),
}
