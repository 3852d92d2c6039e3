"""The Tenotar design in the engine against the plain implementation (tests/plain_tenotar.py).

Every test makes its own small configuration and random weights.  The engine runs the requests in some way of cutting
the work (whole, token by token, in portions down to two tokens, in mixed batches over a pool so small that pages and
state slots are used again) and the logits at every position are compared with the plain implementation's, which knows
no cache.  On the GPU the engine's kernels run, in true 32-bit and in bfloat16; without one the same host logic runs
over the plain operations.
"""

from __future__ import annotations

import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import plain_ops
import plain_tenotar
import tenotar_configs as configs
from test_kafepel import Driver, engine, make_model, tokens_for  # noqa: F401  (the same harness; ``engine`` is a fixture)
from test_nudodra import check

WHERE = ["plain", pytest.param("cuda-float32", marks=pytest.mark.gpu), pytest.param("cuda-bfloat16", marks=pytest.mark.gpu)]
ROOT = Path(__file__).resolve().parent.parent


def expected_of(cfg, tensors, requests):
    return {r: plain_tenotar.forward(cfg, tensors, t) for r, t in requests.items()}


def _loud(tensors):
    """Weights that random draws would leave near nothing, or near one another, made so that leaving them out shows:
    biases, the router's bias, the taps of the convolutions (unequal, some negative), the weights that mix values."""
    g = torch.Generator().manual_seed(99)
    for name, t in tensors.items():
        if name.endswith(".conv"):
            tensors[name] = (torch.randn(t.shape, generator=g) * 0.6).to(t.dtype)
        elif name.endswith("router.b"):
            tensors[name] = (torch.randn(t.shape, generator=g) * 0.8).to(t.dtype)
        elif name.endswith(".b"):
            tensors[name] = (torch.randn(t.shape, generator=g) * 0.3).to(t.dtype)
        elif name.endswith(".vmix"):
            tensors[name] = (torch.rand(t.shape, generator=g) * 0.6 + 0.2).to(t.dtype)


# --------------------------------------------------------------------------------------------- the plain statement
def test_plain_mechanisms_one_by_one():
    """The oracle's own parts against what they are by definition, on inputs where the answer is known."""
    f64 = torch.float64
    x = torch.randn(7, 2, 6, dtype=f64)
    rot = {"dims": 4, "base": 10.0}
    for turn, (a, b) in ((plain_tenotar.rotate_halves, (0, 2)), (plain_tenotar.rotate_neighbours, (0, 1))):
        y = turn(x, rot)
        assert torch.equal(y[0], x[0]) and torch.equal(y[..., 4:], x[..., 4:])  # position 0 and the lanes behind the rotated ones
        assert torch.allclose(y[..., :4].pow(2).sum(-1), x[..., :4].pow(2).sum(-1))  # a rotation keeps lengths
        three = torch.tensor(3.0, dtype=f64)  # the first pair's frequency is 1
        assert torch.allclose(y[3, 0, a], x[3, 0, a] * torch.cos(three) - x[3, 0, b] * torch.sin(three))
        assert torch.allclose(y[3, 0, b], x[3, 0, b] * torch.cos(three) + x[3, 0, a] * torch.sin(three))
    # the second pair of four lanes turns by base^(-2/4)
    y = plain_tenotar.rotate_neighbours(x, rot)
    slow = torch.tensor(5 * 10.0 ** -0.5, dtype=f64)
    assert torch.allclose(y[5, 1, 2], x[5, 1, 2] * torch.cos(slow) - x[5, 1, 3] * torch.sin(slow))
    # masks: a window of three, the same with two kept tokens, blocks of four
    w = plain_tenotar.visible(9, {"size": 3}, "window")
    assert w[8].tolist() == [False] * 6 + [True] * 3 and w[1].tolist() == [True, True] + [False] * 7
    k = plain_tenotar.visible(9, {"size": 3, "keep_first": 2}, "window_keep")
    assert k[8].tolist() == [True, True] + [False] * 4 + [True] * 3 and k[0].tolist() == [True] + [False] * 8
    c = plain_tenotar.visible(9, {"size": 4}, "chunk")
    assert c[5].tolist() == [False] * 4 + [True, True] + [False] * 3 and c[4].tolist() == [False] * 4 + [True] + [False] * 4 and c[8].tolist() == [False] * 8 + [True]
    # the convolution: the newest row meets the last tap, and nothing stands before the sequence
    u = torch.tensor([[1.0], [10.0], [100.0]], dtype=f64)
    y = plain_tenotar.short_convolution(u, torch.tensor([[3.0, 2.0]], dtype=f64))
    assert y[:, 0].tolist() == [2.0, 23.0, 230.0]
    # the router: two of three logits chosen, the weights their softmax alone; an expert with unit matrices is silu(x) * x
    one = torch.ones(1, 1, dtype=f64)
    W = {"router": torch.tensor([[1.0], [2.0], [0.0]], dtype=f64), "router.b": torch.tensor([0.0, 0.0, 5.0], dtype=f64)}
    for e in range(3):
        W.update({f"e{e}.gate": one, f"e{e}.up": one, f"e{e}.down": one * (e + 1)})
    h = torch.tensor([[1.0]], dtype=f64)  # logits 1, 2, 5: experts 2 and 1 with weights softmax(5, 2)
    share = torch.softmax(torch.tensor([5.0, 2.0], dtype=f64), 0)
    unit = torch.sigmoid(torch.tensor(1.0, dtype=f64))
    assert torch.allclose(plain_tenotar.routed(h, W, "", {"router": {"experts": 3, "top": 2}}), (share[0] * 3 + share[1] * 2) * unit)
    # mixed values: the first layer hands on, the second takes its share
    shared = {}
    v1 = plain_tenotar.mix_values(torch.ones(2, 3, dtype=f64), {}, "a.", {"v_mix": True}, shared)
    v2 = plain_tenotar.mix_values(torch.zeros(2, 3, dtype=f64), {"b.vmix": torch.tensor(0.25)}, "b.", {"v_mix": True}, shared)
    assert torch.equal(v1, torch.ones(2, 3, dtype=f64)) and torch.allclose(v2, torch.full((2, 3), 0.25, dtype=f64))


# --------------------------------------------------------------------------------------------- mechanisms alone
ALONE = {
    "window_keeps_first": configs.config([configs.layer(configs.windowed(6, 2, 10, 6, 0.6, 5, keep_first=3, dims=6, base=50.0))], width=32),
    "window_16": configs.config([configs.layer(configs.windowed(4, 2, 32, 16, 0.3, 12, keep_first=1, dims=8))], width=32),
    "blocks_and_convolution": configs.config([configs.layer(configs.blocked(6, 2, 10, 6, 0.7, 6, 4, softcap=2.0))], width=32),
    "blocks_48": configs.config([configs.layer(configs.blocked(8, 2, 48, 48, 0.2, 9, 2))], width=32),
    "latent": configs.config([configs.layer(configs.latent(3, 10, 6, 14, 9, 7, 0.5, 8, base=30.0))], width=32),
    "latent_16": configs.config([configs.layer(configs.latent(4, 16, 16, 32, 48, 16, 0.2, 10))], width=32),
    "mixed_values": configs.config([configs.layer(configs.windowed(2, 1, 8, 12, 0.5, 30, v_mix=True)),
                                    configs.layer(configs.blocked(3, 1, 4, 12, 0.4, 30, 2, v_mix=True)),
                                    configs.layer(configs.windowed(1, 1, 6, 12, 0.4, 30, v_mix=True))], width=32),
    "dense": configs.config([configs.layer(configs.windowed(1, 1, 4, 4, 0.5, 4), configs.dense(40))], width=32),
    "experts": configs.config([configs.layer(configs.windowed(1, 1, 4, 4, 0.5, 4), configs.moe(7, 3, 9, shared=11))], width=32),
    "experts_no_shared": configs.config([configs.layer(configs.windowed(1, 1, 4, 4, 0.5, 4), configs.moe(4, 1, 16))], width=32),
}


@pytest.mark.parametrize("where", WHERE)
@pytest.mark.parametrize("name", sorted(ALONE))
def test_each_mechanism_alone_whole_and_token_by_token(name, where, engine):
    """One to three layers in which one mechanism carries the weight: the whole prompt in one step, and the same tokens
    one by one through the pages and the state."""
    engine(where)
    cfg = ALONE[name]
    model, tensors, dtype = make_model(cfg, 11, where, std=0.2, change=_loud)
    reqs = tokens_for(cfg["vocab"], [37], 5)
    exp = expected_of(cfg, tensors, reqs)
    d = Driver(model, num_pages=24)
    d.run([("r0", reqs["r0"])], end=["r0"])
    check(d.got, exp, dtype, "whole")
    d.got.clear()
    for i, t in enumerate(reqs["r0"]):
        d.run([("r0", [t])], end=["r0"] if i == len(reqs["r0"]) - 1 else [])
    check(d.got, exp, dtype, "token by token")


@pytest.mark.parametrize("where", WHERE)
@pytest.mark.parametrize("name", ["odd", "wide"])
def test_residual_stream_after_every_layer(name, where, engine):
    engine(where)
    cfg = configs.ALL[name]
    model, tensors, dtype = make_model(cfg, 3, where, change=_loud)
    tokens = tokens_for(cfg["vocab"], [19], 2)["r0"]
    _, layers = plain_tenotar.forward(cfg, tensors, tokens, return_layers=True)
    seen = []
    model.layer_probe = lambda i, x: seen.append(x.float().cpu().clone())
    Driver(model, num_pages=16).run([("r0", tokens)], end=["r0"])
    assert len(seen) == len(layers) == len(cfg["layers"])
    tol = 1e-4 if dtype == "float32" else 6e-2
    for i, x in enumerate(seen):
        scale = float(layers[i].abs().max())
        assert float((x - layers[i].float()).abs().max()) <= tol * scale, f"the stream differs after layer {i}"


# --------------------------------------------------------------------------------------------- ways of cutting
@pytest.mark.parametrize("where", WHERE)
@pytest.mark.parametrize("name", sorted(configs.ALL))
def test_ways_of_cutting(name, where, engine):
    """Whole prompts; a prompt then its last tokens one by one; portions of changing size down to two tokens and one;
    the first tokens of a sequence alone."""
    engine(where)
    cfg = configs.ALL[name]
    model, tensors, dtype = make_model(cfg, 7, where, change=_loud)
    reqs = tokens_for(cfg["vocab"], [1, 2, 45, 83], 9)
    exp = expected_of(cfg, tensors, reqs)
    d = Driver(model, num_pages=24)
    for r, t in reqs.items():
        d.run([(r, t)], end=[r])
    check(d.got, exp, dtype, "whole")
    d.got.clear()
    t = reqs["r3"]
    d.run([("r3", t[:40])])
    for i in range(40, len(t)):
        d.run([("r3", [t[i]])], end=["r3"] if i == len(t) - 1 else [])
    check(d.got, exp, dtype, "decode")
    d.got.clear()
    for r in ("r2", "r3"):
        t, i, k = reqs[r], 0, 0
        sizes = (1, 2, 7, 2, 16, 3, 5, 2, 1, 9)
        while i < len(t):
            n = min(sizes[k % len(sizes)], len(t) - i)
            d.run([(r, t[i : i + n])], end=[r] if i + n == len(t) else [])
            i, k = i + n, k + 1
    check(d.got, exp, dtype, "portions")


@pytest.mark.parametrize("where", WHERE)
@pytest.mark.parametrize("name", ["odd", "wide"])
def test_mixed_batches_with_pages_and_slots_used_again(name, where, engine):
    """Up to four unequal requests a step, portions beside single tokens, over a pool of few pages and four state
    slots: every request's logits equal those of the request alone, also on pages and slots that others gave back (a
    slot's rows of the convolution must start at zero again; pages that a window or a block has passed go back early)."""
    engine(where)
    cfg = configs.ALL[name]
    model, tensors, dtype = make_model(cfg, 13, where, change=_loud)
    base = tokens_for(cfg["vocab"], [50, 9, 31, 64, 3, 40], 21)
    exp = expected_of(cfg, tensors, base)
    reqs = {**base, **{r + "#2": t for r, t in base.items()}}  # each once more, on used pages and slots
    prefill = {r: max(1, len(t) - 6) for r, t in reqs.items()}
    d = Driver(model, num_pages=52, page_size=4, max_requests=4)
    waiting, live = list(reqs), {}
    while waiting or live:
        if waiting and len(live) < 4:
            live[waiting.pop(0)] = 0
        entries, end = [], []
        for r, fed in list(live.items()):
            t = reqs[r]
            n = min(7, prefill[r] - fed) if fed < prefill[r] else 1
            n = min(n, len(t) - fed)
            entries.append((r, t[fed : fed + n]))
            live[r] = fed + n
            if live[r] == len(t):
                end.append(r)
                del live[r]
        d.run(entries, end=end)
    assert len({k[0] for k in d.got}) == len(reqs)
    check(d.got, exp, dtype, "mixed")
    assert d.cache.slots.num_used == 0 and all(g.allocator.num_used == 0 for g in d.cache.groups)


def test_pages_behind_windows_and_blocks_go_back_and_kept_ones_stay():
    """The cache manager alone: a group with a window and kept first tokens holds the kept pages and the window's, a group
    of blocks only the newest block's."""
    from llmserve_triton_kernels_b200.cache import CacheManager
    from llmserve_triton_kernels_b200.cache.manager import RELEASED
    from llmserve_triton_kernels_b200.models.plan import LayerRun
    from llmserve_triton_kernels_b200.parts.base import PagedKVSpec

    specs = [PagedKVSpec(1, 4, window=6, keep_first=5), PagedKVSpec(1, 4, chunk=8), PagedKVSpec(1, 4, window=6)]
    cache = CacheManager(specs, [LayerRun(0), LayerRun(1), LayerRun(2)], page_size=4, num_pages=20, max_requests=2, dtype=torch.float32, device="cpu")
    cache.add_request("a")
    cache.reserve([("a", 30)])
    cache.commit([("a", 30)])
    kept, blocks, window = (g.tables["a"] for g in cache.groups)
    # the next query stands at position 30: its window starts at 25 (page 6), its block at 24 (page 6)
    assert [p != RELEASED for p in kept] == [True, True] + [False] * 4 + [True, True]  # tokens 0..4 lie in pages 0 and 1
    assert [p != RELEASED for p in blocks] == [False] * 6 + [True, True]
    assert [p != RELEASED for p in window] == [False] * 6 + [True, True]
    cache.check()
    cache.free_request("a")
    assert all(g.allocator.num_used == 0 for g in cache.groups)


@pytest.mark.parametrize("where", WHERE)
def test_long_decoding_over_pages_windows_and_blocks(where, engine):
    """A short prompt, then many tokens one by one: pages fill one after the other and go back behind windows and blocks,
    the convolution's rows move on at every step, and every window and block edge is passed token by token."""
    engine(where)
    cfg = configs.ODD
    model, tensors, dtype = make_model(cfg, 17, where, change=_loud)
    t = tokens_for(cfg["vocab"], [150], 4)["r0"]
    exp = expected_of(cfg, tensors, {"r0": t})
    d = Driver(model, num_pages=40, page_size=4)
    d.run([("r0", t[:3])])
    for i in range(3, len(t)):
        d.run([("r0", [t[i]])], end=["r0"] if i == len(t) - 1 else [])
    check(d.got, exp, dtype, "long decoding")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_portions(dtype, engine):
    """Prompts of some hundred tokens, whole and in two long portions beside a decoding request; then single tokens
    over a context long enough to be shared out over several CTAs."""
    where = f"cuda-{dtype}"
    engine(where)
    cfg = configs.WIDE
    model, tensors, dtype = make_model(cfg, 23, where, change=_loud)
    reqs = tokens_for(cfg["vocab"], [330, 40], 6)
    exp = expected_of(cfg, tensors, reqs)
    d = Driver(model, num_pages=100, page_size=8)
    d.run([("r0", reqs["r0"])], end=["r0"])
    check(d.got, exp, dtype, "whole")
    d.got.clear()
    d.run([("r1", reqs["r1"][:39])])
    d.run([("r0", reqs["r0"][:150]), ("r1", reqs["r1"][39:])], end=["r1"])
    d.run([("r0", reqs["r0"][150:320])])
    for i in range(320, 330):
        d.run([("r0", [reqs["r0"][i]])], end=["r0"] if i == 329 else [])
    check(d.got, exp, dtype, "two long portions, then single tokens")


# --------------------------------------------------------------------------------------------- faults that random weights would hide
SHARP = {
    # a window of 9 with 3 kept tokens; a window of 5 over 6 kept ones; blocks of 7 with a cap that still lets one key win;
    # a latent window of 11: each alone, with pages of 4 so that every edge falls inside pages and on their borders in turn
    "kept": configs.config([configs.layer(configs.windowed(2, 1, 16, 8, 1.0, 9, keep_first=3, dims=4, base=100.0))], width=32),
    "kept_wide": configs.config([configs.layer(configs.windowed(2, 2, 8, 8, 1.2, 5, keep_first=6))], width=32),
    "blocks": configs.config([configs.layer(configs.blocked(2, 1, 16, 8, 1.0, 7, 3, softcap=12.0))], width=32),
    "latent": configs.config([configs.layer(configs.latent(2, 8, 8, 8, 16, 12, 0.8, 11, base=100.0))], width=32),
}


@pytest.mark.parametrize("where", WHERE)
@pytest.mark.parametrize("name", sorted(SHARP))
def test_keys_at_the_edges_decide(name, where, engine):
    """One attention layer whose queries and keys are scaled up so that scores are sharp: every position leans on one or
    two keys, which over some hundred positions are in turn the key just inside each window or block, the kept tokens,
    keys at page borders and the query's own; the plain statement with a mask that is one key wider or narrower differs
    from the right one by far more than the tolerance.  Prompt in portions that end inside pages, then single tokens."""
    engine(where)
    cfg = SHARP[name]

    def sharp(tensors):
        _loud(tensors)
        for key in ("l0.mix.q.norm", "l0.mix.k.norm", "l0.mix.q.conv", "l0.mix.k.conv", "l0.mix.uq", "l0.mix.uk"):
            if key in tensors:
                tensors[key] = tensors[key] * 2.5

    model, tensors, dtype = make_model(cfg, 29, where, std=0.3, change=sharp)
    t = tokens_for(cfg["vocab"], [260], 12)["r0"]
    exp = expected_of(cfg, tensors, {"r0": t})
    for change in (-1, 1):  # the mask matters in this model: one key more or fewer moves the logits visibly
        other = json.loads(json.dumps(cfg))
        other["layers"][0]["mixer"]["mask"]["size"] += change
        assert float((plain_tenotar.forward(other, tensors, t) - exp["r0"]).abs().max()) > 0.05
    if "keep_first" in cfg["layers"][0]["mixer"]["mask"]:
        other = json.loads(json.dumps(cfg))
        other["layers"][0]["mixer"]["mask"]["keep_first"] -= 1
        assert float((plain_tenotar.forward(other, tensors, t) - exp["r0"]).abs().max()) > 0.05
    d = Driver(model, num_pages=70, page_size=4)
    i = 0
    for n in (3, 126, 2, 70, 39):
        d.run([("r0", t[i : i + n])])
        i += n
    for j in range(i, len(t)):
        d.run([("r0", [t[j]])], end=["r0"] if j == len(t) - 1 else [])
    check(d.got, exp, dtype, "sharp scores")


# --------------------------------------------------------------------------------------------- configuration and plan
def test_configuration_round_trip_and_errors():
    from llmserve_triton_kernels_b200.config import ConfigError, TenotarConfig, architecture_of

    for cfg in configs.ALL.values():
        typed = architecture_of(cfg).config_class.from_dict(cfg)
        assert isinstance(typed, TenotarConfig) and typed.to_dict() == {**cfg, "layers": typed.to_dict()["layers"]}
        assert TenotarConfig.from_dict(typed.to_dict()) == typed
    assert TenotarConfig.from_dict(configs.ODD).value_mix_source() == 0 and TenotarConfig.from_dict(configs.WIDE).value_mix_source() == 0
    bad = json.loads(json.dumps(configs.ODD))
    bad["layers"][2]["mixer"]["vdim"] = 6  # mixed values of another size than the first such layer's
    with pytest.raises(ConfigError, match="v_mix"):
        TenotarConfig.from_dict(bad)
    bad = json.loads(json.dumps(configs.ODD))
    del bad["layers"][1]["mixer"]["q_rank"]
    with pytest.raises(ConfigError, match="q_rank"):
        TenotarConfig.from_dict(bad)
    bad = json.loads(json.dumps(configs.ODD))
    bad["layers"][0]["type"] = "convolution"
    with pytest.raises(ConfigError, match="convolution"):
        TenotarConfig.from_dict(bad)


def test_plan_names_every_tensor_of_the_design():
    model, _, _ = make_model(configs.ODD, 1, "plain")
    names = set(model.tensor_specs())
    for name in ("embed", "head", "final.norm", "l0.norm1", "l0.mix.q.conv", "l0.mix.k.conv", "l0.mix.v.conv", "l0.mix.vmix", "l0.mlp.router",
                 "l0.mlp.router.b", "l0.mlp.e4.gate", "l0.mlp.shared.down", "l1.mix.dq", "l1.mix.dq.norm", "l1.mix.uq", "l1.mix.dkv", "l1.mix.dkv.norm",
                 "l1.mix.uk", "l1.mix.uv", "l1.mix.g", "l1.mlp.gate.b", "l1.mlp.down.b", "l2.mix.q.b", "l2.mix.o.b", "l2.mix.q.norm", "l2.mix.k.norm",
                 "l2.mix.vmix", "l4.mix.vmix"):
        assert name in names, name
    assert "l3.mix.vmix" not in names and "l2.norm2" not in names and "l0.mix.q.b" not in names
    specs = model.tensor_specs()
    assert specs["l1.mix.g"].shape == (3, 40) and specs["l1.mix.uq"].shape == (3 * (6 + 4), 9) and specs["l0.mix.q.conv"].shape == (30, 3)
    # what each layer keeps: pages and a slot for the convolution's rows; a row of latent and rotated key part; pages alone
    kinds = [type(s).__name__ for s in model.cache_specs()]
    assert kinds == ["CompositeSpec", "PagedRowSpec", "PagedKVSpec", "PagedKVSpec", "CompositeSpec"]
    first = model.cache_specs()[0].parts
    assert first[0].chunk == 7 and first[0].window is None and first[1].shape == (2, 30 + 10 + 14)
    assert model.cache_specs()[2].window == 9 and model.cache_specs()[2].keep_first == 3


# --------------------------------------------------------------------------------------------- generation and replay
@pytest.mark.parametrize("where", WHERE)
def test_greedy_generation_through_the_scheduler(where, engine, monkeypatch):
    """``LLM.generate`` with greedy sampling, several prompts at once in portions: every chosen token is the plain
    implementation's choice given the tokens before it (or its logit is within rounding of the best)."""
    engine(where)
    if where == "plain":
        from llmserve_triton_kernels_b200 import ops

        monkeypatch.setattr(ops, "argmax", plain_ops.argmax)
        monkeypatch.setattr(ops, "sample", plain_ops.sample)
    from llmserve_triton_kernels_b200.engine.llm import LLM
    from llmserve_triton_kernels_b200.sampling import SamplingParams
    from llmserve_triton_kernels_b200.weights.random_init import random_tensors

    cfg = configs.ODD
    device, dtype = ("cpu", "float32") if where == "plain" else ("cuda:0", where.split("-")[1])
    llm = LLM(cfg, dtype=dtype, device=device, seed=5, block_size=4, num_blocks=60, max_batch_size=3, chunk_size=6,
              max_num_batched_tokens=16, freeze_gc=False)
    tensors = random_tensors(llm.model.tensor_specs(), 5, 0.02, torch.bfloat16)
    prompts = list(tokens_for(cfg["vocab"], [5, 17, 9, 2], 8).values())
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=12))
    assert [len(o.token_ids) for o in outs] == [12] * 4
    for prompt, o in zip(prompts, outs):
        logits = plain_tenotar.forward(cfg, tensors, prompt + o.token_ids)
        for k, tok in enumerate(o.token_ids):
            row = logits[len(prompt) + k - 1]
            slack = 1e-4 if dtype == "float32" else 0.05
            assert float(row.max() - row[tok]) <= slack * float(row.abs().max()), f"token {k} of a request is not the greedy choice"


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_program_as_a_user_starts_it(dtype, model_folder, tmp_path):
    """``bin/trace_run`` on a model folder: a mixed schedule over a pool that holds less than all requests together."""
    cfg = configs.ODD
    folder = model_folder(cfg, 31, torch.bfloat16, 0.1)
    from llmserve_triton_kernels_b200.weights.loader import read_safetensors

    tensors = read_safetensors(folder)
    reqs = tokens_for(cfg["vocab"], [70, 33, 5], 3)
    exp = expected_of(cfg, tensors, reqs)
    steps = [
        {"step": 0, "entries": [{"id": "r0", "tokens": reqs["r0"][:40], "want": [0, 39]}, {"id": "r2", "tokens": reqs["r2"], "want": [4]}], "end": ["r2"]},
        {"step": 1, "entries": [{"id": "r0", "tokens": reqs["r0"][40:69], "want": []}, {"id": "r1", "tokens": reqs["r1"][:2], "want": [1]}], "end": []},
        {"step": 2, "entries": [{"id": "r0", "tokens": reqs["r0"][69:], "want": [0]}, {"id": "r1", "tokens": reqs["r1"][2:], "want": [0, 30]}], "end": ["r0", "r1"]},
    ]
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype, "--out", str(out), "--max-tokens", "128"],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=900, env={**os.environ})
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [line for line in proc.stdout.splitlines() if line.startswith("done")] == ["done 0", "done 1", "done 2"]
    vocab = cfg["vocab"]
    rows = {n: torch.frombuffer(bytearray((out / f"{n}.f32").read_bytes()), dtype=torch.float32).view(-1, vocab) for n in (0, 1, 2)}
    got = {("r0", 0): rows[0][0], ("r0", 39): rows[0][1], ("r2", 4): rows[0][2], ("r1", 1): rows[1][0], ("r0", 69): rows[2][0], ("r1", 2): rows[2][1],
           ("r1", 32): rows[2][2]}
    check(got, exp, dtype, "replay")
