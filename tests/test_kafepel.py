"""The Kafepel design in the engine against the plain implementation (tests/plain_kafepel.py).

Every test makes its own small configuration and random weights.  The engine runs the requests in some way of
cutting the work (whole, token by token, in portions down to two tokens, in mixed batches over a pool so small that
pages and state slots are used again) and the logits at every position are compared with the plain implementation's,
which knows no cache.  On the GPU the engine's kernels run, in true 32-bit and in bfloat16; without one the same host
logic runs over the plain operations.
"""

from __future__ import annotations

import pytest
import torch

import kafepel_configs as configs
import plain_kafepel
import plain_ops

F32_TOL = 3e-5  # of the root mean square of the row's logits
BF16_TOL = 4e-2

WHERE = ["plain", pytest.param("cuda-float32", marks=pytest.mark.gpu), pytest.param("cuda-bfloat16", marks=pytest.mark.gpu)]


def make_model(cfg_dict: dict, seed: int, where: str, std: float = 0.12, change=None):
    import llmserve_triton_kernels_b200.models  # noqa: F401
    from llmserve_triton_kernels_b200.config import architecture_of
    from llmserve_triton_kernels_b200.models.model import Model
    from llmserve_triton_kernels_b200.weights.random_init import random_tensors

    device, dtype = ("cpu", "float32") if where == "plain" else ("cuda:0", where.split("-")[1])
    arch = architecture_of(cfg_dict)
    config = arch.config_class.from_dict(cfg_dict)
    model = (arch.model_class or Model)(arch.plan(config), getattr(torch, dtype), device)
    tensors = random_tensors(model.tensor_specs(), seed, std, torch.bfloat16)
    if change is not None:
        change(tensors)
    model.bind(tensors)
    return model, tensors, dtype


@pytest.fixture
def engine(monkeypatch):
    """``engine(where)`` patches the plain operations in when there is no GPU to run on."""

    def use(where: str):
        if where == "plain":
            from llmserve_triton_kernels_b200 import ops

            for name in plain_ops.ALL:
                monkeypatch.setattr(ops, name, getattr(plain_ops, name))

    return use


class Driver:
    """Steps of ``[(request, tokens)]`` through the framework's step function; gathers logits by (request, position)."""

    def __init__(self, model, num_pages: int, page_size: int = 4, max_requests: int = 4):
        from llmserve_triton_kernels_b200.cache import CacheManager
        from llmserve_triton_kernels_b200.engine.step import StepFunction

        self.cache = CacheManager(model.cache_specs(), model.plan.schedule, page_size=page_size, num_pages=num_pages,
                                  max_requests=max_requests, dtype=model.dtype, device=model.device)
        self.step = StepFunction(model, self.cache)
        self.fed: dict[str, int] = {}
        self.got: dict[tuple[str, int], torch.Tensor] = {}

    def run(self, entries, end=()):
        from llmserve_triton_kernels_b200.engine.batch import StepEntry

        logits = self.step([StepEntry(r, list(t), list(range(len(t)))) for r, t in entries]).float().cpu()
        row = 0
        for r, t in entries:
            start = self.fed.get(r, 0)
            for i in range(len(t)):
                self.got[(r, start + i)] = logits[row].clone()
                row += 1
            self.fed[r] = start + len(t)
        for r in end:
            self.cache.free_request(r)
            self.fed.pop(r)
        self.cache.check()


def _judge(errors, dtype: str, what: str):
    """``errors``: [(request, position, error)].  In 32-bit every row is within the tolerance.  In bfloat16 a row here
    and there may be beyond it with nothing wrong: where rounding moves a router's choice between two experts of almost
    equal score, or where a branch's output almost cancels before it is normed; at most one row in fifty (or one) may."""
    tol = F32_TOL if dtype == "float32" else BF16_TOL
    over = [(req, pos, err) for req, pos, err in errors if not err <= tol]
    allowed = 0 if dtype == "float32" else max(1, len(errors) // 50)
    if len(over) > allowed:
        req, pos, err = over[0]
        raise AssertionError(f"{what}: {len(over)} of {len(errors)} rows are wrong; the first: request {req!r} position {pos}: error {err:.3e} > {tol:.1e}")


def check(got, expected, dtype: str, what: str = ""):
    errors = []
    for (req, pos), row in sorted(got.items()):
        ref = expected[req.split("#")[0]][pos].float()
        assert torch.isfinite(row).all(), f"{what}: non-finite logits at request {req!r} position {pos}"
        d = row - ref
        errors.append((req, pos, float((d - d.mean()).pow(2).mean().sqrt() / ref.pow(2).mean().sqrt().clamp_min(1e-6))))
    _judge(errors, dtype, what)


def tokens_for(vocab: int, lengths, seed: int):
    g = torch.Generator().manual_seed(seed)
    return {f"r{i}": torch.randint(0, vocab, (n,), generator=g).tolist() for i, n in enumerate(lengths)}


def expected_of(cfg, tensors, requests):
    return {r: plain_kafepel.forward(cfg, tensors, t) for r, t in requests.items()}


# --------------------------------------------------------------------------------------------- the plain statement
def test_plain_mechanisms_one_by_one():
    """The oracle's own parts against what they are by definition, on inputs where the answer is known."""
    T, D = 7, 6
    x = torch.randn(T, 2, D, dtype=torch.float64)
    rot = {"dims": 4, "base": 10.0}
    y = plain_kafepel.rotate(x, rot)
    assert torch.equal(y[0], x[0]) and torch.equal(y[..., 4:], x[..., 4:])  # position 0 and the lanes behind the rotated ones
    assert torch.allclose(y[..., :4].pow(2).sum(-1), x[..., :4].pow(2).sum(-1))  # a rotation keeps lengths
    f = plain_kafepel.frequencies(rot)
    assert torch.allclose(y[3, 0, 0], x[3, 0, 0] * torch.cos(3 * f[0]) - x[3, 0, 2] * torch.sin(3 * f[0]))
    # scaled frequencies: short wavelengths stay, long ones are divided, one in between lies between
    sc = {"dims": 8, "base": 1000.0, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}}
    plain, scaled = plain_kafepel.frequencies({"dims": 8, "base": 1000.0}), plain_kafepel.frequencies(sc)
    assert scaled[0] == plain[0] and torch.allclose(scaled[3], plain[3] / 4.0)
    assert plain[2] / 4.0 < scaled[2] < plain[2] or plain[1] / 4.0 < scaled[1] < plain[1]
    # retention with one head, one lane: a geometric sum
    W = {"q": torch.ones(1, 1, dtype=torch.float64), "k": torch.ones(1, 1, dtype=torch.float64), "v": torch.ones(1, 1, dtype=torch.float64),
         "g": torch.ones(1, 1, dtype=torch.float64), "o": torch.ones(1, 1, dtype=torch.float64)}
    h = torch.ones(5, 1, dtype=torch.float64)
    out = plain_kafepel.retention(h, W, "", {"heads": 1, "dim": 1, "vdim": 1, "decay": [0.5], "rot": {"dims": 0}}, 0.0)
    assert torch.allclose(out[:, 0], torch.full((5,), float(torch.sigmoid(torch.tensor(1.0)))).double())  # o / |o| = 1, times silu(1)


# --------------------------------------------------------------------------------------------- mechanisms alone
ALONE = {
    "attention_heavy": configs.config([configs.layer(configs.left(6, 2, 10, 6, 0.6, dims=6, base=50.0, softcap=3.0, scaling=(2.0, 1.0, 3.0, 20)),
                                                     configs.right(1, 2, 2, (0.5,), dims=2))], width=32),
    "attention_16": configs.config([configs.layer(configs.left(4, 2, 16, 32, 0.4), configs.right(1, 16, 16, (0.9,)))], width=32),
    "retention_heavy": configs.config([configs.layer(configs.left(1, 1, 2, 2, 0.5, dims=2), configs.right(3, 10, 14, (0.8, 0.99, 0.999), dims=6, base=20.0))], width=32),
    "dense": configs.config([configs.layer(configs.left(2, 1, 4, 4, 0.5), configs.right(1, 4, 4, (0.9,)), configs.dense(40))], width=32),
    "routed": configs.config([configs.layer(configs.left(2, 1, 4, 4, 0.5), configs.right(1, 4, 4, (0.9,)), configs.moe(7, 3, 9, 2.5, shared=11))], width=32),
    "routed_no_shared": configs.config([configs.layer(configs.left(2, 1, 4, 4, 0.5), configs.right(1, 4, 4, (0.9,)), configs.moe(4, 1, 16, 0.7))], width=32),
}


def _loud(tensors):
    """Weights that random draws would leave near nothing, made large enough that leaving them out shows."""
    g = torch.Generator().manual_seed(99)
    for name, t in tensors.items():
        if name.endswith(".pb") or name.endswith(".correction"):
            tensors[name] = (torch.randn(t.shape, generator=g) * (1.5 if name.endswith(".pb") else 0.3)).to(t.dtype)
        elif name.endswith(".talk"):
            tensors[name] = (torch.eye(t.shape[0]) * 0.5 + torch.randn(t.shape, generator=g) * 0.6).to(t.dtype)


@pytest.mark.parametrize("where", WHERE)
@pytest.mark.parametrize("name", sorted(ALONE))
def test_each_mechanism_alone_whole_and_token_by_token(name, where, engine):
    """One layer in which one mechanism carries the weight: the whole prompt in one step, and the same tokens one by one
    through the cache and the state."""
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
def test_residual_stream_after_every_layer(where, engine):
    engine(where)
    cfg = configs.ODD
    model, tensors, dtype = make_model(cfg, 3, where, change=_loud)
    tokens = tokens_for(cfg["vocab"], [19], 2)["r0"]
    _, layers = plain_kafepel.forward(cfg, tensors, tokens, return_layers=True)
    seen = []
    model.layer_probe = lambda i, x: seen.append(x.float().cpu().clone())
    Driver(model, num_pages=16).run([("r0", tokens)], end=["r0"])
    assert len(seen) == layers.shape[0] == 3
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
    (a slot's matrix of state must start at zero again)."""
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
    """A short prompt, then many tokens one by one: pages fill one after the other, and a head whose decay is close to
    one carries what the first tokens left to the last."""
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
        logits = plain_kafepel.forward(cfg, tensors, prompt + o.token_ids)
        for k, tok in enumerate(o.token_ids):
            row = logits[len(prompt) + k - 1]
            slack = 1e-4 if dtype == "float32" else 0.05
            assert float(row.max() - row[tok]) <= slack * float(row.abs().max()), f"token {k} of a request is not the greedy choice"


# --------------------------------------------------------------------------------------------- configuration
def test_configuration_is_read_from_the_dictionary_and_written_back():
    from llmserve_triton_kernels_b200.config import ConfigError, KafepelConfig, architecture_of

    for cfg in configs.ALL.values():
        assert architecture_of(cfg).name == "Kafepel"
        c = KafepelConfig.from_dict(cfg)
        assert KafepelConfig.from_dict(c.to_dict()) == c
    with pytest.raises(ConfigError, match="convolution"):
        KafepelConfig.from_dict({**configs.ODD, "layers": [{"type": "convolution", "mixer": {}, "mlp": None}]})
    bad = configs.config([configs.layer(configs.left(3, 2, 4, 4, 0.5), configs.right(1, 4, 4, (0.9,)))])
    with pytest.raises(ConfigError, match="kv_heads"):
        KafepelConfig.from_dict(bad)
    bad = configs.config([configs.layer(configs.left(2, 1, 4, 4, 0.5), configs.right(2, 4, 4, (0.9,)))])
    with pytest.raises(ConfigError, match="decay"):
        KafepelConfig.from_dict(bad)
    bad = configs.config([configs.layer(configs.left(2, 1, 4, 4, 0.5), configs.right(1, 4, 4, (0.9,)), configs.moe(3, 4, 8))])
    with pytest.raises(ConfigError, match="top"):
        KafepelConfig.from_dict(bad)


def test_plan_names_every_tensor_and_keeps_pages_and_state_per_layer():
    import llmserve_triton_kernels_b200.models  # noqa: F401
    from llmserve_triton_kernels_b200.config import KafepelConfig
    from llmserve_triton_kernels_b200.models.kafepel import kafepel_plan
    from llmserve_triton_kernels_b200.models.model import Model
    from llmserve_triton_kernels_b200.parts.base import CompositeSpec, PagedKVSpec, StateSpec

    plan = kafepel_plan(KafepelConfig.from_dict(configs.ODD))
    assert plan.embedding_scale == 3.0 and [r.layer for r in plan.schedule] == [0, 1, 2]
    model = Model(plan, torch.float32, "cpu")
    names = set(model.tensor_specs())
    assert {"embed", "head", "final.norm", "l0.norm1", "l0.norm2", "l0.mix.left.q.norm", "l0.mix.left.talk", "l0.mix.left.pb", "l0.mix.left.out",
            "l0.mix.right.g", "l0.mix.right.out", "l0.mlp.gate", "l1.mlp.router", "l1.mlp.correction", "l1.mlp.e4.down", "l1.mlp.shared.sg"} <= names
    assert "l2.norm2" not in names and "l1.mlp.e5.up" not in names
    specs = model.cache_specs()
    assert all(isinstance(s, CompositeSpec) for s in specs)
    assert specs[0].parts == (PagedKVSpec(1, 10, None), StateSpec((2, 6, 10), torch.float32))
    assert model.graph_safe


def test_cache_manager_holds_both_halves_of_a_side_by_side_mixer():
    """Pages and state slots of composite entries: reserved, viewed, freed and used again like those of plain ones."""
    import llmserve_triton_kernels_b200.models  # noqa: F401
    from llmserve_triton_kernels_b200.cache import CacheManager, CompositeView
    from llmserve_triton_kernels_b200.parts.base import CompositeSpec, PagedKVSpec, StateSpec
    from llmserve_triton_kernels_b200.models.plan import LayerRun

    specs = [CompositeSpec((PagedKVSpec(2, 8), StateSpec((3, 4, 5)))), CompositeSpec((PagedKVSpec(2, 8), StateSpec((1, 2, 2)))), StateSpec((7,))]
    cache = CacheManager(specs, [LayerRun(0), LayerRun(1), LayerRun(2)], page_size=4, num_pages=6, max_requests=2, dtype=torch.float32, device="cpu")
    assert len(cache.groups) == 1 and cache.groups[0].pool.shape[0] == 2  # both layers' pages in one group, a plane each
    cache.add_request("a")
    cache.reserve([("a", 9)])
    tables, slots = cache.step_tables([("a", 9)])
    views = cache.views([(torch.from_numpy(t), torch.from_numpy(s)) for t, s in tables], torch.from_numpy(slots), slots.tolist())
    assert isinstance(views[0], CompositeView) and views[0].parts[0].pool.shape == (6, 2, 2, 4, 8) and views[0].parts[1].states.shape == (2, 3, 4, 5)
    assert views[1].parts[1].states.shape == (2, 1, 2, 2) and views[2].states.shape == (2, 7)
    views[0].parts[1].states[slots[0]].fill_(3.0)
    cache.commit([("a", 9)])
    cache.free_request("a")
    cache.add_request("b")  # takes the slot that "a" gave back: its state is zero again
    assert float(views[0].parts[1].states[cache.slot_of["b"]].abs().sum()) == 0.0
    cache.check()


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
    done, rows = {}, {}
    for (req, pos), row in got.items():
        key = tuple(flat[req])
        if key not in done:
            done[key] = plain_kafepel.forward(cfg, tensors, flat[req])
        rows[(req, pos)] = (torch.from_numpy(row.copy()), done[key][pos])
    assert rows
    errors = []
    for (req, pos), (row, ref) in sorted(rows.items()):
        d = row.double() - ref
        errors.append((req, pos, float((d - d.mean()).pow(2).mean().sqrt() / ref.pow(2).mean().sqrt().clamp_min(1e-6))))
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
