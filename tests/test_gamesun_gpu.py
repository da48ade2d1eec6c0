"""Gamesun through the framework against the plain implementation (``tests/plain/gamesun_plain.py``): each mechanism
alone, whole prompts, token-by-token decoding through the captured steps, portions down to two tokens, unequal
requests in one batch against each alone, state slots and pages that are given back and used again, long decoding
(windows pass over decoded tokens), and greedy generation through the engine's own entry point and scheduler.
Four small configurations that differ in every size (``gamesun_configs``); weights are drawn so that attention is
peaked and states remember dozens of tokens, and the tests of the mechanisms alone first show, with the plain
implementation, that a window one token off or a state that forgot its past would be seen.

Tolerances are derived: the float32 engine may be off by a multiple of what float32 arithmetic costs the plain
implementation itself (float32 against float64); the bfloat16 engine by 3 times what rounding the activations to
bfloat16, where a bfloat16 run stores them, costs the plain implementation."""

import functools

import pytest
import torch

from clockwork_b200 import EngineConfig, ops
from clockwork_b200.config import PartSpec
from clockwork_b200.engine import LLMEngine
from clockwork_b200.engine.trace import TraceSession
from clockwork_b200.parts import ResidualStream, build_part
from clockwork_b200.sampling import SamplingParams
from clockwork_b200.weights.loader import make_fetch
from tests.gamesun_configs import CONFIGS, write_model
from tests.gamesun_configs import tokens_for as raw_tokens_for
from tests.gpu_tools import DEV, PartHarness
from tests.plain import gamesun_plain as plain
from tests.plain.qwen2_plain import read_model_dir
from tests.trace_tools import cut

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    return {name: write_model(tmp_path_factory.mktemp(f"gamesun_{name}"), name, seed=5 + i) for i, name in enumerate(sorted(CONFIGS))}


@pytest.fixture(scope="module")
def oracle(dirs):
    """(name, tokens) -> (float64 logits [T, V], what float32 costs, what bfloat16 storage costs)."""
    weights = {name: read_model_dir(folder, dtype=torch.float64) for name, folder in dirs.items()}

    @functools.lru_cache(maxsize=None)
    def get(name, tokens):
        config, w = weights[name]
        exact = plain.forward(config, w, list(tokens), dtype=torch.float64)
        single = plain.forward(config, w, list(tokens), dtype=torch.float32).double()
        rounded = plain.forward(config, w, list(tokens), dtype=torch.float64, rnd=plain.to_bfloat16_and_back)
        return exact, float((single - exact).abs().max()), float((rounded - exact).abs().max())

    return get


_first_tokens: dict = {}


def tokens_for(config, length, salt=0):
    """A prompt that starts with a token whose answer at position 0 rounding cannot flip (at position 0 a head of the
    linear attention with a norm per head puts out sign(q.k) n(v); see ``plain.first_position_margin``).  The first
    token is chosen with the plain implementation, once per configuration."""
    tokens = raw_tokens_for(config, length, salt)
    first = _first_tokens.get(config["vocab"])
    if first is not None:
        tokens[0] = first
    return tokens


@pytest.fixture(scope="module", autouse=True)
def steady_first_tokens(dirs):
    for name, folder in dirs.items():
        config, w = read_model_dir(folder, dtype=torch.float64)
        _first_tokens[config["vocab"]] = plain.steady_first_token(config, w)
    yield
    _first_tokens.clear()


def check(got, name, tokens, dtype, oracle, first=0):
    exact, cost32, cost16 = oracle(name, tuple(tokens))
    diff = (got.double().cpu() - exact[first : first + got.shape[0]]).abs()
    allowed = 30 * cost32 + 1e-5 if dtype == "float32" else 3 * cost16
    worst = float(diff.max())
    assert worst <= allowed, f"{name} {dtype}: off by {worst:.3g} at position {first + int(diff.max(1).values.argmax())}, allowed {allowed:.3g}"


class Replay:
    """Steps through ``TraceSession`` (what ``bin/trace_run`` runs), logits wanted everywhere."""

    def __init__(self, folder, name, dtype, max_tokens, **kw):
        self.session = TraceSession(folder, dtype, max_tokens, page_size=CONFIGS[name][1], **kw)
        self.logits: dict[str, list] = {}
        self.n = 0

    def step(self, portions: dict, end=()):
        record = {"step": self.n, "end": list(end),
                  "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))} for rid, toks in portions.items()]}
        self.n += 1
        out, _ = self.session.run_step(record)
        row = 0
        for rid, toks in portions.items():
            self.logits.setdefault(rid, []).append(torch.from_numpy(out[row : row + len(toks)].copy()))
            row += len(toks)

    def of(self, rid):
        return torch.cat(self.logits[rid])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_whole_prompt(name, dtype, dirs, oracle):
    tokens = tokens_for(CONFIGS[name][0], 75, salt=1)
    run = Replay(dirs[name], name, dtype, 128)
    run.step({"a": tokens}, end=["a"])
    check(run.of("a"), name, tokens, dtype, oracle)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_prefill_then_token_by_token(name, dtype, dirs, oracle):
    """The decoded tokens run through the captured single-token steps; the first tokens of a sequence too (a prompt
    of one token).  70 tokens pass every window but the longest."""
    tokens = tokens_for(CONFIGS[name][0], 70, salt=2)
    for prompt in (9, 1):
        run = Replay(dirs[name], name, dtype, 128)
        run.step({"a": tokens[:prompt]})
        for t in tokens[prompt:]:
            run.step({"a": [t]})
        assert run.session.uses_graphs
        check(run.of("a"), name, tokens, dtype, oracle)


@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_portions_of_many_sizes(name, dtype, graphs, dirs, oracle):
    """Cuts in the middle of pages and of windows, portions of two and three tokens, of one page, longer than a window."""
    tokens = tokens_for(CONFIGS[name][0], 90, salt=3)
    for sizes in ([2, 3, 1, 7, 2, 16, 5, 4], [37, 2, 2, 2, 30, 1, 1, 3]):
        run = Replay(dirs[name], name, dtype, 128, graphs=graphs)
        for portion in cut(tokens, sizes):
            run.step({"a": portion})
        check(run.of("a"), name, tokens, dtype, oracle)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_unequal_requests_in_one_batch_against_each_alone(name, dtype, dirs, oracle):
    config = CONFIGS[name][0]
    prompts = {"p": tokens_for(config, 61, salt=4), "q": tokens_for(config, 23, salt=5), "r": tokens_for(config, 40, salt=6),
               "s": tokens_for(config, 9, salt=7)}
    plans = {"p": [17, 2, 1, 1, 30, 1, 1, 1, 7], "q": [1, 1, 1, 5, 1, 2, 12], "r": [40], "s": [2, 1, 1, 1, 1, 1, 1, 1]}
    cuts = {rid: cut(toks, plans[rid]) for rid, toks in prompts.items()}
    together = Replay(dirs[name], name, dtype, 4 * 64)
    for i in range(max(len(c) for c in cuts.values())):
        step = {rid: c[i] for rid, c in cuts.items() if i < len(c)}
        together.step(step, end=[rid for rid, c in cuts.items() if i == len(c) - 1])
    for rid, toks in prompts.items():
        alone = Replay(dirs[name], name, dtype, 64)
        for portion in cuts[rid]:
            alone.step({rid: portion})
        if dtype == "float32":  # a row's result does not depend on the rest of the batch at all
            assert torch.equal(together.of(rid), alone.of(rid)), rid
        check(together.of(rid), name, toks, dtype, oracle)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_slots_and_pages_given_back_and_used_again(name, dtype, dirs, oracle):
    """Ten requests through four state slots and a pool of pages for 4 x 64 tokens: a request that takes a slot or a
    page that another one left starts from zero state and sees none of the other's keys."""
    config = CONFIGS[name][0]
    run = Replay(dirs[name], name, dtype, 4 * 64)
    prompts = {f"r{i}": tokens_for(config, 20 + 4 * i, salt=20 + i) for i in range(10)}
    waiting, live, at = list(prompts), [], {}
    while waiting or live:
        while waiting and len(live) < 4:
            live.append(waiting.pop(0))
            at[live[-1]] = 0
        step, done = {}, []
        for k, rid in enumerate(live):
            n = min([13, 1, 2, 5][(k + at[rid]) % 4], len(prompts[rid]) - at[rid])
            step[rid] = prompts[rid][at[rid] : at[rid] + n]
            at[rid] += n
            if at[rid] == len(prompts[rid]):
                done.append(rid)
        run.step(step, end=done)
        live = [rid for rid in live if rid not in done]
    run.session.cache.check_invariants()
    assert not run.session.cache.requests and run.session.cache.state.num_free == 4
    for rid, toks in prompts.items():
        check(run.of(rid), name, toks, dtype, oracle)


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_in_a_pool_that_only_windows_make_enough(dtype, dirs, oracle):
    """300 decoded tokens behind a short prompt: every window passes over decoded tokens, states are carried 300
    times, and the pages behind the windows go back to the pool while the request runs."""
    name = "A"
    tokens = tokens_for(CONFIGS[name][0], 320, salt=8)
    run = Replay(dirs[name], name, dtype, 320)
    run.step({"a": tokens[:20]})
    for t in tokens[20:]:
        run.step({"a": [t]})
    req = run.session.cache.get("a")
    assert all(sum(p >= 0 for p in table) <= 50 // 4 + 2 for table in req.tables)
    check(run.of("a"), name, tokens, dtype, oracle)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_greedy_generation_through_the_engine(name, dtype, dirs):
    """The engine's own entry point and scheduler: prompts cut under a small token budget, several requests at once."""
    config, page, _ = CONFIGS[name]
    cfg = EngineConfig.defaults(str(dirs[name]), dtype=dtype, block_size=page, num_blocks=256, max_model_len=256, max_num_seqs=4,
                                max_num_batched_tokens=24)
    engine = LLMEngine(cfg)
    prompts = [tokens_for(config, n, salt=30 + n) for n in (5, 31, 18, 1, 44)]
    outs = engine.generate(prompts, SamplingParams(max_tokens=12, ignore_eos=True))
    _, w = read_model_dir(dirs[name], dtype=torch.float64)
    for prompt, out in zip(prompts, outs):
        got = list(out.token_ids)
        logits = plain.forward(config, w, prompt + got, dtype=torch.float64)
        single = plain.forward(config, w, prompt + got, dtype=torch.float32).double()
        rounded = plain.forward(config, w, prompt + got, dtype=torch.float64, rnd=plain.to_bfloat16_and_back)
        # every token is within rounding of the best one, given the engine's own history
        yard = 60 * float((single - logits).abs().max()) + 2e-5 if dtype == "float32" else 6 * float((rounded - logits).abs().max())
        for i, token in enumerate(got):
            row = logits[len(prompt) + i - 1]
            assert float(row.max() - row[token]) <= yard
        if dtype == "float32" and all(float(r.topk(2).values.diff().abs()) > yard for r in logits[len(prompt) - 1 : -1]):
            assert got == plain.greedy_generate(config, w, prompt, 12)


# ---- every mechanism alone ----------------------------------------------------------------------------

def part_with_weights(category, spec, prefix, dtype, tensors):
    part = build_part(category, spec, prefix, dtype, DEV)
    decls = {d.name: d for d in part.tensor_decls()}
    assert set(decls) == set(tensors), (sorted(decls), sorted(tensors))
    part.load_weights(make_fetch(lambda n: tensors[n], decls, dtype, DEV))
    return part


def run_mixer(part, x, portions, page_size=4, num_pages=128):
    """The mixer's contribution for every row of ``x`` [T, W], fed in portions through a cache of its own."""
    harness = PartHarness({0: part.cache_need()}, part.dtype, num_pages=num_pages, page_size=page_size, slots=2)
    out, at = [], 0
    for n in portions:
        prepared = harness.prepare({"a": n})
        stream = ResidualStream(torch.zeros((n, x.shape[1]), dtype=torch.float32, device=DEV))
        stream.push(part.forward(prepared.ctx, x[at : at + n].to(DEV, part.dtype).contiguous(), prepared.ctx.views[0], stream))
        stream.flush()
        harness.commit(prepared)
        out.append(stream.residual.cpu())
        at += n
    assert at == x.shape[0]
    return torch.cat(out)


def draw(gen, shape, scale=1.0, shift=0.0):
    return (shift + scale * torch.randn(shape, generator=gen)).to(torch.bfloat16).float()


def assert_close(got, want, what, rel=3e-5):
    """float32 arithmetic against float64: a few units of float32 rounding of the largest value, per term summed."""
    worst, allowed = float((got.double() - want).abs().max()), 2e-4 + rel * float(want.abs().max())
    assert worst <= allowed, f"{what}: off by {worst:.3g}, allowed {allowed:.3g}"


def attention_tensors(gen, w, heads, kv_heads, dim, vdim, gated):
    t = {"m.q": draw(gen, (heads * dim, w), 0.5), "m.k": draw(gen, (kv_heads * dim, w), 0.5), "m.v": draw(gen, (kv_heads * vdim, w), 0.3),
         "m.o": draw(gen, (w, heads * vdim), 0.2)}
    if gated:
        t.update({"m.q.b": draw(gen, (heads * dim,), 0.3), "m.k.b": draw(gen, (kv_heads * dim,), 0.3), "m.v.b": draw(gen, (kv_heads * vdim,), 0.3),
                  "m.o.b": draw(gen, (w,), 0.3), "m.talk": (torch.eye(heads) + 0.4 * torch.randn(heads, heads, generator=gen)).to(torch.bfloat16).float(),
                  "m.pb": draw(gen, (heads,), 1.0, -1.0)})
    else:
        t["m.temp"] = draw(gen, (heads,), 0.4, 1.2)
    return t


def attention_spec(w, heads, kv_heads, dim, vdim, window, scale, gated):
    return PartSpec("window_attention", dict(hidden_size=w, heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, window=window, scale=scale,
                                             bias=gated, talk=gated, head_bias=gated, head_scale=not gated,
                                             weights="sigmoid" if gated else "softmax"))


@pytest.mark.parametrize("gated", [False, True])
@pytest.mark.parametrize("heads, kv_heads, dim, vdim, window, page", [(4, 2, 24, 12, 21, 4), (3, 1, 16, 40, 7, 8), (6, 6, 8, 8, 130, 16),
                                                                     (2, 1, 40, 72, 1, 4), (5, 5, 12, 20, 64, 16), (33, 11, 8, 4, 10, 4)])
def test_window_attention_alone(gated, heads, kv_heads, dim, vdim, window, page):
    """Both kinds of weights over 300 positions, whole, token by token and in portions that cut pages and windows.
    First the plain implementation shows that the edge counts: with a window one token shorter or longer the
    result moves by far more than the test allows."""
    gen = torch.Generator().manual_seed(heads * 100 + window)
    w, scale = 48, 0.4
    t = attention_tensors(gen, w, heads, kv_heads, dim, vdim, gated)
    wd = {k: v.double() for k, v in t.items()}
    x = draw(gen, (300, w))
    fn = plain.sigmoid_window_attention if gated else plain.softmax_window_attention
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, mask={"size": window})
    want = fn(x.double(), wd, "m", m)
    for other in (window - 1, window + 1):
        if other >= 1:
            assert float((fn(x.double(), wd, "m", dict(m, mask={"size": other})) - want).abs().max()) > 0.05
    part = part_with_weights("mixer", attention_spec(w, heads, kv_heads, dim, vdim, window, scale, gated), "m", torch.float32, t)
    # few enough pages that the ones behind the window must come back for the run to finish
    pages = (max(window, 131) + 2 * page) // page + 4
    for portions in ([131, 169], [1] * 300, [2, 3, 1, 1, 9, 2, 5, 41, 100, 1, 1, 1, 131, 2], [page - 1, 2, page, 1, 300 - 2 * page - 2][:5]):
        if sum(portions) != 300 or min(portions) < 1:
            continue
        got = run_mixer(part, x, portions, page_size=page, num_pages=pages + max(portions) // page)
        assert_close(got, want, portions)


def test_one_key_that_stands_out_at_the_edge_of_the_window():
    """A query and two keys are made so that one score towers over all others: the key at the far edge of the window
    takes the whole softmax, the key one further back must not be seen at all, in a prompt and in decoding."""
    heads, kv_heads, dim, vdim, window, w = 2, 1, 16, 8, 37, 32
    gen = torch.Generator().manual_seed(9)
    t = attention_tensors(gen, w, heads, kv_heads, dim, vdim, gated=False)
    t["m.temp"] = torch.ones(heads)
    x = draw(gen, (120, w), 0.05)
    probe, inside, outside = 100, 100 - window + 1, 100 - window
    x[probe, 3] += 40.0    # every query channel reads coordinate 3, every key channel coordinate 5
    x[inside, 5] += 40.0
    x[outside, 5] += 80.0  # would win if it were visible
    t["m.q"][:, 3] = 0.5
    t["m.k"][:, 5] = 0.5
    wd = {k: v.double() for k, v in t.items()}
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=1.0, mask={"size": window})
    want = plain.softmax_window_attention(x.double(), wd, "m", m)
    v_inside = (x[inside].double() @ wd["m.v"].T).repeat(heads) @ wd["m.o"].T
    assert float((want[probe] - v_inside).abs().max()) < 1e-6  # the edge key alone
    part = part_with_weights("mixer", attention_spec(w, heads, kv_heads, dim, vdim, window, 1.0, False), "m", torch.float32, t)
    for portions in ([120], [probe, 1, 19], [outside + 1, 20, 100 - outside - 21 + 1, 19]):
        got = run_mixer(part, x, portions, page_size=8)
        assert_close(got, want, portions)


def test_windows_cut_in_parts_when_a_step_has_few_tokens():
    """bfloat16 steps of a few tokens cut windows longer than 256 across thread blocks; the parts add up to the same."""
    from clockwork_b200.ops import window as window_ops

    heads, kv_heads, dim, vdim, window, w = 4, 2, 32, 48, 300, 64
    assert window_ops.window_parts(1, window, torch.bfloat16) > 1 and window_ops.window_parts(1, window, torch.float32) == 1
    gen = torch.Generator().manual_seed(4)
    x = draw(gen, (420, w))
    for gated in (False, True):
        t = attention_tensors(gen, w, heads, kv_heads, dim, vdim, gated)
        wd = {k: v.double() for k, v in t.items()}
        fn = plain.sigmoid_window_attention if gated else plain.softmax_window_attention
        m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=0.3, mask={"size": window})
        want = fn(x.double(), wd, "m", m)
        yard = float((fn(x.double(), wd, "m", m, rnd=plain.to_bfloat16_and_back) - want).abs().max())
        part = part_with_weights("mixer", attention_spec(w, heads, kv_heads, dim, vdim, window, 0.3, gated), "m", torch.bfloat16, t)
        cut_up = run_mixer(part, x, [150] + [1] * 200 + [3, 67], page_size=16)
        whole = run_mixer(part, x, [420], page_size=16)
        assert float((cut_up.double() - want).abs().max()) <= 3 * yard
        # the same bfloat16 queries, keys and values either way: what is left is the rounding of the weighted sums
        assert float((cut_up - whole).abs().max()) <= 0.02 * float(want.abs().max())


@pytest.mark.parametrize("gated", [False, True])
@pytest.mark.parametrize("heads, kv_heads, dim, vdim, window, page", [(4, 2, 32, 48, 21, 4), (16, 4, 64, 64, 70, 16), (6, 3, 64, 96, 44, 16),
                                                                     (3, 1, 16, 40, 7, 8), (4, 4, 16, 24, 33, 8), (4, 2, 96, 160, 100, 16),
                                                                     (2, 1, 128, 128, 300, 16)])
def test_window_attention_on_tensor_cores(gated, heads, kv_heads, dim, vdim, window, page):
    """The bfloat16 kernel on the tensor cores against the CUDA-core one and against the plain implementation: tiles of
    16 rows that end in the middle of a portion, single tokens, windows that start in the middle of a tile of keys,
    windows cut in parts (the last size)."""
    from clockwork_b200.ops import window as window_ops

    gen = torch.Generator().manual_seed(heads * 10 + window)
    w, scale = 64, 0.25
    t = attention_tensors(gen, w, heads, kv_heads, dim, vdim, gated)
    for name in ("m.q", "m.k"):
        t[name] = (t[name] * 0.6).to(torch.bfloat16).float()
    wd = {k: v.double() for k, v in t.items()}
    x = draw(gen, (330, w))
    fn = plain.sigmoid_window_attention if gated else plain.softmax_window_attention
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, mask={"size": window})
    want = fn(x.double(), wd, "m", m)
    yard = float((fn(x.double(), wd, "m", m, rnd=plain.to_bfloat16_and_back) - want).abs().max())
    part = part_with_weights("mixer", attention_spec(w, heads, kv_heads, dim, vdim, window, scale, gated), "m", torch.bfloat16, t)
    for portions in ([330], [100, 1, 1, 1, 17, 16, 15, 33, 1, 145], [5] + [1] * 325):
        outs = []
        for on in (True, False):
            window_ops.set_tensor_cores(on)
            try:
                outs.append(run_mixer(part, x, portions, page_size=page, num_pages=512))
            finally:
                window_ops.set_tensor_cores(True)
        fast, slow = outs
        assert float((fast.double() - want).abs().max()) <= 3 * yard, portions
        assert float((slow.double() - want).abs().max()) <= 3 * yard, portions
        assert float((fast - slow).abs().max()) <= yard, portions


@pytest.mark.parametrize("heads, dim, vdim, rank, tau", [(3, 20, 12, 5, 8.0), (1, 64, 8, 8, 1.0), (2, 72, 40, 16, 30.0), (5, 8, 130, 3, 4.0)])
def test_gated_linear_attention_alone(heads, dim, vdim, rank, tau):
    gen = torch.Generator().manual_seed(dim)
    w = 40
    t = {"m.q": draw(gen, (heads * dim, w), 0.2), "m.k": draw(gen, (heads * dim, w), 0.2), "m.v": draw(gen, (heads * vdim, w), 0.2),
         "m.g": draw(gen, (heads * vdim, w), 0.2), "m.o": draw(gen, (w, heads * vdim), 0.1), "m.a1": draw(gen, (rank, w), 0.3),
         "m.a2": draw(gen, (heads * dim, rank), 0.5), "m.a2.b": draw(gen, (heads * dim,), 1.0, 2.0), "m.norm": draw(gen, (vdim,), 0.2, 1.0)}
    cfg = dict(heads=heads, dim=dim, vdim=vdim, tau=tau)
    part = part_with_weights("mixer", PartSpec("gated_linear", dict(cfg, hidden_size=w, eps=1e-5)), "m", torch.float32, t)
    x = draw(gen, (150, w))
    wd = {k: v.double() for k, v in t.items()}
    want = plain.channel_decay_mixer(x.double(), wd, "m", cfg, 1e-5)
    if tau > 1:  # the state remembers: without the first hundred tokens the rest comes out differently
        assert float((plain.channel_decay_mixer(x.double()[100:], wd, "m", cfg, 1e-5) - want[100:]).abs().max()) > 0.02
    for portions in ([150], [1] * 150, [2, 1, 3, 2, 42, 17, 16, 1, 66]):
        got = run_mixer(part, x, portions)
        assert_close(got, want, portions)


@pytest.mark.parametrize("heads, dim, vdim, decay", [(3, 20, 12, [0.6, 0.97, 1.0]), (1, 64, 8, [0.99]), (2, 8, 130, [0.9, 0.999]),
                                                     (4, 16, 16, [0.5, 0.75, 0.9, 0.95])])
def test_decay_linear_attention_alone(heads, dim, vdim, decay):
    gen = torch.Generator().manual_seed(vdim)
    w = 40
    t = {"m.q": draw(gen, (heads * dim, w), 0.3), "m.k": draw(gen, (heads * dim, w), 0.3), "m.v": draw(gen, (heads * vdim, w), 0.3),
         "m.g": draw(gen, (heads * vdim, w), 0.2), "m.o": draw(gen, (w, heads * vdim), 0.1), "m.norm": draw(gen, (heads * vdim,), 0.2, 1.0)}
    cfg = dict(heads=heads, dim=dim, vdim=vdim, decay=decay)
    part = part_with_weights("mixer", PartSpec("decay_linear", dict(cfg, hidden_size=w, eps=1e-5)), "m", torch.float32, t)
    x = draw(gen, (150, w))
    wd = {k: v.double() for k, v in t.items()}
    want = plain.head_decay_mixer(x.double(), wd, "m", cfg, 1e-5)
    if max(decay) > 0.95:
        assert float((plain.head_decay_mixer(x.double()[100:], wd, "m", cfg, 1e-5) - want[100:]).abs().max()) > 0.02
    for portions in ([150], [1] * 150, [2, 1, 3, 2, 42, 17, 16, 1, 66]):
        got = run_mixer(part, x, portions)
        assert_close(got, want, portions)


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_two_mixers_on_two_streams_change_nothing(dtype, dirs):
    """The left mixer's kernels run on a second stream beside the right one's: the same bits as one after the other,
    in prompts, portions and captured single-token steps."""
    from clockwork_b200.parts.side_by_side import SideBySide

    name = "D"
    tokens = tokens_for(CONFIGS[name][0], 120, salt=15)
    results = []
    for concurrent in (True, False):
        SideBySide.concurrent = concurrent
        try:
            run = Replay(dirs[name], name, dtype, 256)
            for portion in cut(tokens, [70, 3, 17, 1, 1, 1, 1, 1, 25]):
                run.step({"a": portion})
            results.append(run.of("a"))
        finally:
            SideBySide.concurrent = True
    assert torch.equal(results[0], results[1])


@pytest.mark.parametrize("kind", ["parallel", "parallel_2"])
def test_two_mixers_side_by_side_alone(kind):
    """Pages for the one and a state slot for the other in the same layer; each output normed over the width."""
    from tests.gamesun_configs import CONFIG_A, draw_weights

    layer = 0 if kind == "parallel" else 1
    config = CONFIG_A
    assert config["layers"][layer]["type"] == kind
    weights = draw_weights(config, 5, seed=2)
    prefix = f"l{layer}.mix"
    t = {k: v.float() for k, v in weights.items() if k.startswith(prefix + ".")}
    from clockwork_b200.config.registry import spec_from_raw

    spec = spec_from_raw(config).layers[layer].mixer
    part = part_with_weights("mixer", spec, prefix, torch.float32, t)
    gen = torch.Generator().manual_seed(6)
    x = draw(gen, (60, config["width"]))
    want = plain.side_by_side(x.double(), {k: v.double() for k, v in t.items()}, prefix, kind, config["layers"][layer]["mixer"], 1e-5)
    for portions in ([60], [1] * 60, [7, 2, 30, 1, 20]):
        got = run_mixer(part, x, portions)
        assert_close(got, want, portions)


def test_scaled_embedding_with_position_vectors():
    """Positions far from zero: float32 angles against the plain implementation's float64 ones, within what the
    float32 product position * frequency costs."""
    width, count = 72, 40
    gen = torch.Generator().manual_seed(8)
    x = draw(gen, (count, width))
    positions = torch.tensor([0, 1, 2, 3, 17, 255, 256, 1000, 4095, 30000] * 4, dtype=torch.int32)
    part = build_part("position", PartSpec("sinusoidal_absolute", {"size": width, "base": 10000.0}), "", torch.float32, DEV)
    got = x.to(DEV).contiguous()
    part.add_to_embedding(got, positions.to(DEV), 3.5)
    table = plain.position_vectors(30001, width, torch.float64)
    want = x.double() * 3.5 + table[positions.long()]
    err = (got.cpu().double() - want).abs()
    assert float(err[positions < 300].max()) < 5e-5 and float(err.max()) < 30000 * 2e-7


def test_swiglu_with_short_names_and_a_layer_without_feed_forward(dirs):
    gen = torch.Generator().manual_seed(1)
    w, ff = 40, 100
    t = {"f.gate": draw(gen, (ff, w), 0.3), "f.up": draw(gen, (ff, w), 0.3), "f.down": draw(gen, (w, ff), 0.2)}
    part = part_with_weights("ffn", PartSpec("swiglu", dict(hidden_size=w, intermediate_size=ff, names=("gate", "up", "down"))), "f",
                             torch.float32, t)
    x = draw(gen, (19, w), 2.0)
    harness = PartHarness({}, torch.float32)
    prepared = harness.prepare({"a": 19})
    stream = ResidualStream(torch.zeros((19, w), dtype=torch.float32, device=DEV))
    stream.push(part.forward(prepared.ctx, x.to(DEV).contiguous(), stream))
    stream.flush()
    want = plain.gated_ff(x.double(), {k: v.double() for k, v in t.items()}, "f")
    assert float((stream.residual.cpu().double() - want).abs().max()) < 1e-4
    from clockwork_b200.engine import load_model

    model = load_model(dirs["A"], "float32", DEV)  # layer 1 of configuration A has no feed-forward
    assert model.blocks[1].ffn is None and len(model.blocks[1].parts()) == 2 and len(model.blocks[0].parts()) == 4


@pytest.mark.timeout(600)
def test_a_step_at_layer_sizes_of_a_real_model():
    """Four layers at 2,048 width with windows of 1,024 and 4,096: a prompt portion and single-token steps through the
    captured graphs agree with the same steps launched kernel by kernel."""
    from clockwork_b200.cache import CacheManager
    from clockwork_b200.cli import shape_config
    from clockwork_b200.engine import ModelRunner, StepEntry, random_model

    raw = shape_config("gamesun-2k", 4)
    model = random_model(raw, seed=3, dtype="bfloat16", device=DEV)
    prompt = tokens_for({"vocab": raw["vocab"]}, 1300, salt=9)
    tail = tokens_for({"vocab": raw["vocab"]}, 3, salt=10)
    results = []
    for graphs in (True, False):
        cache = CacheManager(model.cache_needs(), num_pages=128, page_size=16, dtype=model.dtype, device=DEV, num_state_slots=2)
        runner = ModelRunner(model, cache)
        if graphs:
            assert runner.enable_graphs(max_ctx=2048, max_batch=2)
        cache.open("a")
        rows = [runner.step([StepEntry("a", prompt, [len(prompt) - 1])]).float().cpu()]
        for t in tail:
            entry = [StepEntry("a", [t], [0])]
            if graphs:
                runner.decode_with_graph(entry, None)
                rows.append(runner.last_graph.logits[:1].float().cpu())
            else:
                rows.append(runner.step(entry).float().cpu())
        runner.check_status()
        assert not graphs or runner.graphs
        results.append(torch.cat(rows))
    assert torch.isfinite(results[0]).all()
    scale = float(results[1].abs().max())
    assert float((results[0] - results[1]).abs().max()) <= 0.02 * scale
