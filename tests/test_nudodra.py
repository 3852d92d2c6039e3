"""The Nudodra design in the engine against the plain implementation (tests/plain_nudodra.py).

Every test makes its own small configuration and random weights.  The engine runs the requests in some way of cutting
the work (whole, token by token, in portions down to two tokens, in mixed batches over a pool so small that pages and
state slots are used again) and the logits at every position are compared with the plain implementation's, which knows
no cache.  On the GPU the engine's kernels run, in true 32-bit and in bfloat16; without one the same host logic runs
over the plain operations.
"""

from __future__ import annotations

import pytest
import torch

import nudodra_configs as configs
import plain_nudodra
import plain_ops
from test_kafepel import BF16_TOL, F32_TOL, Driver, engine, make_model, tokens_for  # noqa: F401  (the same harness; ``engine`` is a fixture)

WHERE = ["plain", pytest.param("cuda-float32", marks=pytest.mark.gpu), pytest.param("cuda-bfloat16", marks=pytest.mark.gpu)]


def _judge(errors, dtype: str, what: str):
    """``errors``: [(request, position, error)].  In 32-bit every row is within the tolerance: that is the test of the
    mechanisms and of the cache.  In bfloat16 the same host logic runs over the 16-bit kernels, and rounding alone leaves
    a median error near 1e-2 with a tail (a stream's copies that nearly cancel, a branch that enters times two, sharp
    scores): no row may be beyond 0.15, and at most one row in ten beyond the tolerance."""
    tol = F32_TOL if dtype == "float32" else BF16_TOL
    over = [(req, pos, err) for req, pos, err in errors if not err <= tol]
    far = [(req, pos, err) for req, pos, err in errors if not err <= 0.15]
    allowed = 0 if dtype == "float32" else max(1, len(errors) // 10)
    if len(over) > allowed or far:
        req, pos, err = (far or over)[0]
        raise AssertionError(f"{what}: {len(over)} of {len(errors)} rows are wrong; the first: request {req!r} position {pos}: error {err:.3e} > {tol:.1e}")


def check(got, expected, dtype: str, what: str = ""):
    errors = []
    scale = _scale_of([expected[req.split("#")[0]][pos] for req, pos in got], dtype)
    for (req, pos), row in sorted(got.items()):
        ref = expected[req.split("#")[0]][pos].float()
        assert torch.isfinite(row).all(), f"{what}: non-finite logits at request {req!r} position {pos}"
        d = row - ref
        errors.append((req, pos, float((d - d.mean()).pow(2).mean().sqrt() / ref.pow(2).mean().sqrt().clamp_min(scale))))
    _judge(errors, dtype, what)


def _scale_of(rows, dtype: str) -> float:
    """What a row's error is divided by, at least.  In 32-bit: next to nothing, so every row is measured against its own
    size.  In bfloat16 a row's rounding error follows the size of the activations it came through, not its own size: a row
    whose logits happen to be small is measured against the root mean square of all rows compared."""
    if dtype == "float32":
        return 1e-6
    return float(torch.stack([r.double().pow(2).mean() for r in rows]).mean().sqrt())


def expected_of(cfg, tensors, requests):
    return {r: plain_nudodra.forward(cfg, tensors, t) for r, t in requests.items()}


def _loud(tensors):
    """Weights that random draws would leave near nothing, made large enough that leaving them out shows: biases, sinks,
    the decays' bias (so that channels forget at very different rates), and the weights around the stream's copies."""
    g = torch.Generator().manual_seed(99)
    for name, t in tensors.items():
        if name.endswith(".sink"):
            tensors[name] = (torch.randn(t.shape, generator=g) * 1.5 + 1.0).to(t.dtype)
        elif name.endswith(".a2.b"):
            tensors[name] = (torch.randn(t.shape, generator=g) * 2.5 + 2.0).to(t.dtype)
        elif name.endswith(".b"):
            tensors[name] = (torch.randn(t.shape, generator=g) * 0.3).to(t.dtype)
        elif ".hc" in name and name.endswith(".mix"):
            tensors[name] = (torch.eye(t.shape[0]) * 0.8 + torch.randn(t.shape, generator=g) * 0.15).to(t.dtype)
        elif ".hc" in name:
            tensors[name] = (1.0 + torch.randn(t.shape, generator=g) * 0.25).to(t.dtype)


# --------------------------------------------------------------------------------------------- the plain statement
def test_plain_mechanisms_one_by_one():
    """The oracle's own parts against what they are by definition, on inputs where the answer is known."""
    f64 = torch.float64
    x = torch.randn(7, 2, 6, dtype=f64)
    y = plain_nudodra.rotate(x, {"dims": 4, "base": 10.0})
    assert torch.equal(y[0], x[0]) and torch.equal(y[..., 4:], x[..., 4:])  # position 0 and the lanes behind the rotated ones
    assert torch.allclose(y[..., :4].pow(2).sum(-1), x[..., :4].pow(2).sum(-1))  # a rotation keeps lengths
    f0 = 10.0 ** 0.0
    assert torch.allclose(y[3, 0, 0], x[3, 0, 0] * torch.cos(torch.tensor(3 * f0, dtype=f64)) - x[3, 0, 2] * torch.sin(torch.tensor(3 * f0, dtype=f64)))
    # the queries' factor: 1 until position every - 2, then a step at every multiple of ``every``
    t = plain_nudodra.query_temperature(9, {"coef": 2.0, "every": 4})
    assert t[:3].tolist() == [1.0, 1.0, 1.0] and torch.allclose(t[3:7], torch.full((4,), 1 + 2 * torch.log(torch.tensor(2.0)).item(), dtype=f64))
    assert torch.allclose(t[7], 1 + 2 * torch.log(torch.tensor(3.0, dtype=f64)))
    # a sink of score 0 beside one key of score 0 halves that key's weight; a sink far below changes nothing
    s = torch.zeros(1, 1, 1, dtype=f64)
    assert torch.allclose(plain_nudodra.softmax_rows(s, torch.zeros(1, dtype=f64)), torch.full((1, 1, 1), 0.5, dtype=f64))
    assert torch.allclose(plain_nudodra.softmax_rows(s, torch.full((1,), -80.0, dtype=f64)), torch.ones(1, 1, 1, dtype=f64))
    # gated linear attention with one head, one lane, logits 0 and tau 1: a geometric sum of ratio 1/2
    one = torch.ones(1, 1, dtype=f64)
    W = {"q": one, "k": one, "v": one, "g": one, "o": one, "norm": torch.ones(1, dtype=f64), "a1": one, "a2": 0 * one, "a2.b": torch.zeros(1, dtype=f64)}
    h = torch.ones(5, 1, dtype=f64)
    out = plain_nudodra.gated_linear_attention(h, W, "", {"heads": 1, "dim": 1, "vdim": 1, "tau": 1.0}, 0.0)
    assert torch.allclose(out[:, 0], torch.full((5,), float(torch.sigmoid(torch.tensor(1.0))), dtype=f64))  # o / |o| = 1, times silu(1)
    # an expert: the gate is bounded from above only, the up product on both sides
    W = {"gate": torch.tensor([[1.0]], dtype=f64), "up": torch.tensor([[1.0]], dtype=f64), "down": torch.tensor([[1.0]], dtype=f64)}
    big, small = plain_nudodra.expert(torch.tensor([[50.0]], dtype=f64), W, "", 2.0), plain_nudodra.expert(torch.tensor([[-50.0]], dtype=f64), W, "", 2.0)
    assert torch.allclose(big, 2.0 * torch.sigmoid(torch.tensor(1.702 * 2.0, dtype=f64)) * 3.0) and abs(float(small)) < 1e-30
    # hyper-connections with identity mixing and unit weights on one copy are the plain residual sum
    X = torch.randn(1, 4, 3, dtype=f64)
    W = {"in": torch.ones(1, dtype=f64), "out": torch.ones(1, dtype=f64), "mix": torch.ones(1, 1, dtype=f64)}
    assert torch.allclose(plain_nudodra.hyper_sublayer(X, W, "", torch.ones(3, dtype=f64), 0.0, lambda h: 2 * h)[0], X[0] + 2 * plain_nudodra.rms(X[0], 0.0))


# --------------------------------------------------------------------------------------------- mechanisms alone
_TINY_RIGHT = configs.right(1, 2, 2, 2.0, rank=1)
_TINY_LEFT = configs.left(1, 1, 2, 0.5, dims=2)
ALONE = {
    "sink_attention": configs.config([configs.parallel_layer(configs.left(6, 2, 10, 0.6, dims=6, base=50.0), _TINY_RIGHT, 1.0, 0.05)], width=32),
    "sink_attention_16": configs.config([configs.parallel_layer(configs.left(4, 2, 32, 0.3, dims=8), _TINY_RIGHT, 1.2, 0.05)], width=32, streams=1),
    "gated_linear": configs.config([configs.parallel_layer(_TINY_LEFT, configs.right(3, 10, 14, 3.0, rank=4), 0.05, 1.4)], width=32),
    "gated_linear_wide": configs.config([configs.parallel_layer(_TINY_LEFT, configs.right(2, 40, 70, 20.0, rank=2), 0.05, 0.9)], width=32, streams=None),
    "attention": configs.config([configs.attention_layer(configs.attention(6, 2, 10, 6, 0.5, coef=0.9, every=4))], width=32),
    "attention_48": configs.config([configs.attention_layer(configs.attention(8, 2, 48, 48, 0.2, coef=0.3, every=8))], width=32),
    "shared_pages": configs.config([configs.attention_layer(configs.attention(2, 1, 8, 4, 0.5, coef=0.5, every=4)),
                                    configs.attention_layer(configs.attention(4, 1, 8, 4, 0.4, coef=0.8, every=2, kv_from=0))], width=32),
    "experts": configs.config([configs.attention_layer(configs.attention(1, 1, 4, 4, 0.5), configs.moe(7, 3, 9, 0.3, shared=11, shared_limit=0.15))], width=32),
    "experts_no_shared": configs.config([configs.attention_layer(configs.attention(1, 1, 4, 4, 0.5), configs.moe(4, 1, 16, 0.5))], width=32, streams=5),
}


@pytest.mark.parametrize("where", WHERE)
@pytest.mark.parametrize("name", sorted(ALONE))
def test_each_mechanism_alone_whole_and_token_by_token(name, where, engine):
    """One or two layers in which one mechanism carries the weight: the whole prompt in one step, and the same tokens one
    by one through the cache and the state."""
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
@pytest.mark.parametrize("name", ["odd", "plain"])
def test_residual_stream_after_every_layer(name, where, engine):
    engine(where)
    cfg = configs.ALL[name]
    model, tensors, dtype = make_model(cfg, 3, where, change=_loud)
    tokens = tokens_for(cfg["vocab"], [19], 2)["r0"]
    _, layers = plain_nudodra.forward(cfg, tensors, tokens, return_layers=True)
    seen = []
    model.layer_probe = lambda i, x: seen.append(x.float().cpu().clone())
    Driver(model, num_pages=16).run([("r0", tokens)], end=["r0"])
    assert len(seen) == layers.shape[0] == len(cfg["layers"])
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
    slots: every request's logits equal those of the request alone, also on pages and slots that others gave back
    (a slot's matrix of state must start at zero again, and a layer that reads another's pages must read its own request's)."""
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


@pytest.mark.parametrize("where", WHERE)
def test_long_decoding_over_pages_with_a_state_carried_far(where, engine):
    """A short prompt, then many tokens one by one: pages fill one after the other, the queries' factor steps up several
    times, and a head whose channels hardly decay (a large tau) carries what the first tokens left to the last."""
    engine(where)
    cfg = configs.ONES
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
@pytest.mark.parametrize("where", WHERE)
def test_a_key_far_back_decides_and_the_sink_counts(where, engine):
    """One attention layer whose query and key weights are scaled up so that scores are sharp: every position then leans
    on few keys, often far back, and a sink close to the largest scores takes a visible share of the weight.  Prompt of
    some hundred tokens in portions that end inside pages, then single tokens."""
    engine(where)
    cfg = configs.config([configs.parallel_layer(configs.left(2, 1, 16, 1.0, dims=4, base=100.0), _TINY_RIGHT, 1.0, 0.01)], width=32)

    def sharp(tensors):
        _loud(tensors)
        for name in ("l0.mix.left.q.norm", "l0.mix.left.k.norm"):
            tensors[name] = tensors[name] * 2.0
        tensors["l0.mix.left.sink"] = torch.tensor([4.0, -3.0]).to(tensors["l0.mix.left.sink"].dtype)

    model, tensors, dtype = make_model(cfg, 29, where, std=0.3, change=sharp)
    t = tokens_for(cfg["vocab"], [260], 12)["r0"]
    exp = expected_of(cfg, tensors, {"r0": t})
    no_sink = dict(tensors)
    no_sink["l0.mix.left.sink"] = torch.full((2,), -60.0)
    assert float((plain_nudodra.forward(cfg, no_sink, t) - exp["r0"]).abs().max()) > 0.05  # the sink matters in this model
    d = Driver(model, num_pages=70, page_size=4)
    i = 0
    for n in (3, 126, 2, 70, 39):
        d.run([("r0", t[i : i + n])])
        i += n
    for j in range(i, len(t)):
        d.run([("r0", [t[j]])], end=["r0"] if j == len(t) - 1 else [])
    check(d.got, exp, dtype, "sharp scores")


# --------------------------------------------------------------------------------------------- generation
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
        logits = plain_nudodra.forward(cfg, tensors, prompt + o.token_ids)
        for k, tok in enumerate(o.token_ids):
            row = logits[len(prompt) + k - 1]
            slack = 1e-4 if dtype == "float32" else 0.05
            assert float(row.max() - row[tok]) <= slack * float(row.abs().max()), f"token {k} of a request is not the greedy choice"


# --------------------------------------------------------------------------------------------- configuration
def test_configuration_is_read_from_the_dictionary_and_written_back():
    from llmserve_triton_kernels_b200.config import ConfigError, NudodraConfig, architecture_of

    for cfg in configs.ALL.values():
        assert architecture_of(cfg).name == "Nudodra"
        c = NudodraConfig.from_dict(cfg)
        assert NudodraConfig.from_dict(c.to_dict()) == c
    assert NudodraConfig.from_dict(configs.PLAIN).streams is None and "streams" not in NudodraConfig.from_dict(configs.PLAIN).to_dict()
    with pytest.raises(ConfigError, match="convolution"):
        NudodraConfig.from_dict({**configs.ODD, "layers": [{"type": "convolution", "mixer": {}, "mlp": None}]})
    with pytest.raises(ConfigError, match="kv_heads"):
        NudodraConfig.from_dict(configs.config([configs.attention_layer(configs.attention(3, 2, 4, 4, 0.5))]))
    with pytest.raises(ConfigError, match="kv_from"):
        NudodraConfig.from_dict(configs.config([configs.attention_layer(configs.attention(2, 1, 4, 4, 0.5, kv_from=0))]))
    with pytest.raises(ConfigError, match="whose keys and values it reads"):  # the named layer has other heads
        NudodraConfig.from_dict(configs.config([configs.attention_layer(configs.attention(2, 1, 4, 4, 0.5)), configs.attention_layer(configs.attention(2, 2, 4, 4, 0.5, kv_from=0))]))
    with pytest.raises(ConfigError, match="top"):
        NudodraConfig.from_dict(configs.config([configs.attention_layer(configs.attention(2, 1, 4, 4, 0.5), configs.moe(3, 4, 8, 1.0))]))
    with pytest.raises(ConfigError, match="tau"):
        NudodraConfig.from_dict(configs.config([configs.parallel_layer(configs.left(1, 1, 4, 0.5), configs.right(1, 4, 4, 0.0), 1.0, 1.0)]))
    with pytest.raises(ConfigError, match="streams"):
        NudodraConfig.from_dict(configs.config([configs.attention_layer(configs.attention(2, 1, 4, 4, 0.5))], streams=0))


def test_plan_names_every_tensor_and_shares_pages_between_entries():
    import llmserve_triton_kernels_b200.models  # noqa: F401
    from llmserve_triton_kernels_b200.config import NudodraConfig
    from llmserve_triton_kernels_b200.models.model import Model
    from llmserve_triton_kernels_b200.models.nudodra import nudodra_plan
    from llmserve_triton_kernels_b200.parts.base import CompositeSpec, PagedKVSpec, StateSpec

    plan = nudodra_plan(NudodraConfig.from_dict(configs.ODD))
    assert plan.streams == 3 and [(r.layer, r.cache_of) for r in plan.schedule] == [(0, None), (1, None), (2, 1), (3, None), (4, 1)]
    model = Model(plan, torch.float32, "cpu")
    names = set(model.tensor_specs())
    assert {"embed", "head", "final.norm", "l0.norm1", "l0.norm2", "l0.mix.left.q.b", "l0.mix.left.k.norm", "l0.mix.left.sink", "l0.mix.right.a1",
            "l0.mix.right.a2.b", "l0.mix.right.norm", "l0.mlp.table", "l0.mlp.e4.gate", "l0.mlp.shared.down", "l0.hc1.mix", "l0.hc2.in",
            "l1.mix.q.b", "l1.mix.v.b", "l1.mix.g", "l2.mix.q", "l2.mix.g", "l2.hc1.out"} <= names
    for absent in ("l0.mix.left.v", "l0.mix.left.out", "l2.mix.k", "l2.mix.v.b", "l2.norm2", "l2.hc2.in", "l1.mlp.shared.gate", "l0.mlp.e5.up", "l1.mlp.router"):
        assert absent not in names, absent
    specs = model.cache_specs()
    assert isinstance(specs[0], CompositeSpec) and specs[0].parts == (PagedKVSpec(1, 10, None), StateSpec((2, 6, 10), torch.float32))
    assert specs[1] == PagedKVSpec(2, 14, None) and specs[2] is None and specs[4] is None
    assert model.graph_safe
    # a checkpoint says the inner size of the decay's products itself; a random model takes a stand-in
    assert model.tensor_specs()["l3.mix.right.a1"].shape == (-1, 40) and model.tensor_specs()["l0.mix.right.a1"].shape == (3, 40)


def test_a_checkpoint_gives_the_decay_its_inner_size(tmp_path, engine):
    """``a1`` and ``a2`` of any inner size load when they agree, and are refused when they do not."""
    import llmserve_triton_kernels_b200.models  # noqa: F401
    from llmserve_triton_kernels_b200.models.load import load_model
    from safetensors.torch import save_file
    import json

    engine("plain")
    cfg = configs.config([configs.parallel_layer(configs.left(1, 1, 4, 0.5), configs.right(2, 4, 6, 3.0), 1.0, 1.0)], width=16)
    model, tensors, _ = make_model(cfg, 1, "plain")
    g = torch.Generator().manual_seed(2)
    tensors["l0.mix.right.a1"] = (torch.randn(5, 16, generator=g) * 0.2).to(torch.bfloat16)
    tensors["l0.mix.right.a2"] = (torch.randn(8, 5, generator=g) * 0.2).to(torch.bfloat16)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(tmp_path / "model.safetensors"))
    loaded, _ = load_model(tmp_path, "float32", "cpu")
    toks = tokens_for(cfg["vocab"], [9], 3)["r0"]
    d = Driver(loaded, num_pages=8)
    d.run([("r0", toks)], end=["r0"])
    check(d.got, expected_of(cfg, tensors, {"r0": toks}), "float32", "inner size 5")
    tensors["l0.mix.right.a2"] = tensors["l0.mix.right.a2"][:, :4].contiguous()
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(tmp_path / "model.safetensors"))
    with pytest.raises(ValueError, match="inner size"):
        load_model(tmp_path, "float32", "cpu")


# --------------------------------------------------------------------------------------------- the replay program
def _replay_trace(cfg, seed=31):
    import trace_tools

    reqs = tokens_for(cfg["vocab"], [41, 6, 75, 20, 33], seed)
    trace = trace_tools.Trace()
    flat = {}
    for r, t in list(reqs.items())[:2]:
        for tag, make in (("w", trace_tools.whole), ("d", lambda n, x: trace_tools.decode_tail(n, x, tail=5)), ("p", trace_tools.portions)):
            trace.extend(make(f"{tag}.{r}", t))
            flat[f"{tag}.{r}"] = t
    both = {**{f"m.{r}": t for r, t in reqs.items()}, **{f"m.{r}'": t for r, t in reqs.items()}}
    trace.extend(trace_tools.mixed(both, {k: max(1, len(v) - 4) for k, v in both.items()}, chunk=9, live=4))
    flat.update(both)
    return trace, flat


def _check_replay(got, cfg, tensors, flat, dtype):
    done, errors = {}, []
    assert got
    for req in {req for req, _ in got}:
        if tuple(flat[req]) not in done:
            done[tuple(flat[req])] = plain_nudodra.forward(cfg, tensors, flat[req])
    scale = _scale_of([done[tuple(flat[req])][pos] for req, pos in got], dtype)
    for (req, pos), row in sorted(got.items()):
        ref = done[tuple(flat[req])][pos]
        d = torch.from_numpy(row.copy()).double() - ref
        errors.append((req, pos, float((d - d.mean()).pow(2).mean().sqrt() / ref.pow(2).mean().sqrt().clamp_min(scale))))
    _judge(errors, dtype, "replay")


def _model_folder(cfg, tmp_path, seed=3, std=0.12):
    import llmserve_triton_kernels_b200.models  # noqa: F401
    from llmserve_triton_kernels_b200.config import architecture_of
    from llmserve_triton_kernels_b200.weights import write_random_model
    from llmserve_triton_kernels_b200.weights.loader import read_safetensors

    folder = write_random_model(tmp_path / "model", architecture_of(cfg).config_class.from_dict(cfg), seed=seed, std=std)
    return folder, read_safetensors(folder)


def test_replay_program_host_side(tmp_path, engine):
    """A model folder of the design through the replay program in this process, over the plain operations: the folder's
    config.json picks the model class, steps come as JSON lines, logits go to files, pages and slots are used again."""
    import trace_tools

    engine("plain")
    cfg = configs.ODD
    folder, tensors = _model_folder(cfg, tmp_path)
    trace, flat = _replay_trace(cfg)
    got = trace_tools.run_trace_inprocess(folder, "float32", trace, tmp_path / "out", device="cpu", page_size=4)
    _check_replay(got, cfg, tensors, flat, "float32")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["odd", "wide"])
def test_replay_program_as_a_user_starts_it(name, dtype, tmp_path):
    import trace_tools

    cfg = configs.ALL[name]
    folder, tensors = _model_folder(cfg, tmp_path)
    trace, flat = _replay_trace(cfg)
    got = trace_tools.run_trace(folder, dtype, trace, tmp_path / "out")
    _check_replay(got, cfg, tensors, flat, dtype)
