"""Rapitar through the framework against the plain implementation (``tests/plain/rapitar_plain.py``):
each mixer and feed-forward alone, whole prompts, token-by-token decoding through the captured steps,
portions down to two tokens, unequal requests in one batch against each alone, state slots and pages
that are given back and used again, long decoding, and greedy generation through the engine's own
entry point and scheduler.  Three small configurations that differ in every size (``rapitar_configs``);
weights are drawn so that attention is peaked, sinks count, and states remember dozens of tokens.

Tolerances are derived: the float32 engine may be off by a multiple of what float32 arithmetic costs the
plain implementation itself (float32 against float64); the bfloat16 engine by 3 times what rounding the
activations to bfloat16, where a bfloat16 run stores them, costs the plain implementation."""

import functools

import pytest
import torch

from clockwork_b200 import EngineConfig
from clockwork_b200.config import PartSpec
from clockwork_b200.engine import LLMEngine, load_model
from clockwork_b200.engine.trace import TraceSession
from clockwork_b200.parts import ResidualStream, build_part
from clockwork_b200.sampling import SamplingParams
from clockwork_b200.weights.loader import make_fetch
from tests.gpu_tools import DEV, PartHarness
from tests.plain import rapitar_plain as plain
from tests.plain.qwen2_plain import read_model_dir
from tests.rapitar_configs import CONFIGS, tokens_for, write_model
from tests.trace_tools import cut

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    return {name: write_model(tmp_path_factory.mktemp(f"rapitar_{name}"), name, seed=11 + i) for i, name in enumerate(sorted(CONFIGS))}


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
    """The decoded tokens run through the captured single-token steps; the first tokens of a sequence too (a
    prompt of one token)."""
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
    """Cuts in the middle of pages, portions of two and three tokens, of one page, and longer than the taps of the
    short convolution or shorter."""
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
    """Ten requests through four state slots and a pool of pages for 4 x 64 tokens: a request that takes a slot
    or a page that another one left starts from zero state and sees none of the other's keys."""
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
def test_long_decoding(dtype, dirs, oracle):
    """300 decoded tokens behind a short prompt: contexts across many pages, states carried 300 times."""
    name = "A"
    tokens = tokens_for(CONFIGS[name][0], 320, salt=8)
    run = Replay(dirs[name], name, dtype, 320)
    run.step({"a": tokens[:20]})
    for t in tokens[20:]:
        run.step({"a": [t]})
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
        if dtype == "float32":
            assert got == plain.greedy_generate(config, w, prompt, 12)
        else:  # every token is within rounding of the best one, given the engine's own history
            logits = plain.forward(config, w, prompt + got, dtype=torch.float64)
            rounded = plain.forward(config, w, prompt + got, dtype=torch.float64, rnd=plain.to_bfloat16_and_back)
            yard = float((rounded - logits).abs().max())
            for i, token in enumerate(got):
                row = logits[len(prompt) + i - 1]
                assert float(row.max() - row[token]) <= 6 * yard


# ---- every mechanism alone ----------------------------------------------------------------------------

def part_with_weights(category, spec, prefix, dtype, tensors):
    part = build_part(category, spec, prefix, dtype, DEV)
    decls = {d.name: d for d in part.tensor_decls()}
    assert set(decls) == set(tensors), (sorted(decls), sorted(tensors))
    part.load_weights(make_fetch(lambda n: tensors[n], decls, dtype, DEV))
    return part


def run_mixer(part, x, portions, page_size=4):
    """The mixer's contribution for every row of ``x`` [T, W], fed in portions through a cache of its own."""
    harness = PartHarness({0: part.cache_need()}, part.dtype, num_pages=128, page_size=page_size, slots=2)
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


@pytest.mark.parametrize("heads, vdim, state, groups, taps, parts", [(4, 12, 20, 2, 3, 2), (1, 40, 9, 1, 1, 1), (6, 8, 130, 3, 6, 4)])
def test_mamba2_alone(heads, vdim, state, groups, taps, parts):
    gen = torch.Generator().manual_seed(heads)
    w, inner, gn = 32, heads * vdim, groups * state
    t = {"m.in": draw(gen, (2 * inner + 2 * gn + heads, w), 0.2), "m.conv": draw(gen, (inner + 2 * gn, taps), 0.5),
         "m.conv.b": draw(gen, (inner + 2 * gn,), 0.3), "m.dt_bias": draw(gen, (heads,), 0.5, -2.0), "m.A_log": draw(gen, (heads,), 0.5, -1.0),
         "m.D": draw(gen, (heads,), 0.3, 1.0), "m.norm": draw(gen, (inner,), 0.2, 1.0), "m.o": draw(gen, (w, inner), 0.1)}
    cfg = dict(heads=heads, vdim=vdim, state=state, groups=groups, conv=taps, norm_groups=parts)
    spec = PartSpec("mamba2", dict(cfg, hidden_size=w, eps=1e-5))
    part = part_with_weights("mixer", spec, "m", torch.float32, t)
    x = draw(gen, (64, w))
    want = plain.mamba2_mixer(x.double(), {k: v.double() for k, v in t.items()}, "m", cfg, 1e-5)
    for portions in ([64], [1] * 64, [2, 3, 1, 1, 9, 2, 5, 41], [taps, max(taps - 1, 1), 64 - taps - max(taps - 1, 1)]):
        got = run_mixer(part, x, portions)
        assert float((got.double() - want).abs().max()) < 2e-4, portions


@pytest.mark.parametrize("heads, dim, rank", [(3, 20, 5), (1, 64, 8), (2, 72, 16)])
def test_wkv_alone(heads, dim, rank):
    gen = torch.Generator().manual_seed(dim)
    w, a = 40, heads * dim
    t = {f"m.mu.{s}": torch.rand((w,), generator=gen).to(torch.bfloat16).float() for s in "rkvgw"}
    t.update({f"m.{s}": draw(gen, (a, w), 0.15) for s in "rkvg"})
    t.update({"m.w1": draw(gen, (rank, w), 0.3), "m.w2": draw(gen, (a, rank), 0.5), "m.w0": draw(gen, (a,), 0.7, -3.0),
              "m.u": draw(gen, (heads, dim), 0.5), "m.norm": draw(gen, (a,), 0.2, 1.0), "m.o": draw(gen, (w, a), 0.1)})
    cfg = dict(heads=heads, dim=dim)
    part = part_with_weights("mixer", PartSpec("wkv", dict(cfg, hidden_size=w, eps=1e-5)), "m", torch.float32, t)
    x = draw(gen, (50, w))
    want = plain.wkv_mixer(x.double(), {k: v.double() for k, v in t.items()}, "m", cfg, 1e-5)
    for portions in ([50], [1] * 50, [2, 1, 3, 2, 42]):
        got = run_mixer(part, x, portions)
        assert float((got.double() - want).abs().max()) < 2e-4, portions


@pytest.mark.parametrize("heads, dim, rot, vdim, rank, q_rank, page", [(3, 24, 8, 20, 40, 24, 4), (1, 16, 16, 16, 16, 8, 16), (5, 8, 4, 12, 136, 32, 8),
                                                                      (6, 16, 2, 8, 24, 16, 4)])
def test_latent_attention_alone(heads, dim, rot, vdim, rank, q_rank, page):
    """Peaked attention over 300 keys: most queries put most of their weight on one key far back, somewhere in
    another page; and sinks large enough to take a visible share."""
    gen = torch.Generator().manual_seed(rank)
    w = 48
    t = {"m.dq": draw(gen, (q_rank, w), 0.3), "m.dq.norm": draw(gen, (q_rank,), 0.2, 1.0), "m.uq": draw(gen, (heads * (dim + rot), q_rank), 1.2),
         "m.dkv": draw(gen, (rank + rot, w), 0.6), "m.dkv.norm": draw(gen, (rank,), 0.2, 1.0), "m.uk": draw(gen, (heads * dim, rank), 0.4),
         "m.uv": draw(gen, (heads * vdim, rank), 0.3), "m.sink": draw(gen, (heads,), 1.5, 2.0), "m.g": draw(gen, (heads * vdim, w), 0.3),
         "m.o": draw(gen, (w, heads * vdim), 0.2)}
    cfg = dict(heads=heads, dim=dim, rot_dim=rot, vdim=vdim, kv_rank=rank, q_rank=q_rank, scale=0.4, rot={"base": 300.0, "dims": rot})
    spec = PartSpec("latent_attention", dict(hidden_size=w, heads=heads, dim=dim, rot_dim=rot, vdim=vdim, kv_rank=rank, q_rank=q_rank,
                                             scale=0.4, rope_base=300.0, eps=1e-5))
    part = part_with_weights("mixer", spec, "m", torch.float32, t)
    x = draw(gen, (300, w))
    wd = {k: v.double() for k, v in t.items()}
    want = plain.latent_attention_mixer(x.double(), wd, "m", cfg, 1e-5)
    without_sink = plain.latent_attention_mixer(x.double(), dict(wd, **{"m.sink": torch.full((heads,), -1e9).double()}), "m", cfg, 1e-5)
    assert float((want - without_sink).abs().max()) > 0.05  # the sink matters here
    short = plain.latent_attention_mixer(x.double()[100:], wd, "m", cfg, 1e-5, positions=torch.arange(100, 300))
    assert float((want[100:] - short).abs().max()) > 0.05  # and so do keys more than a hundred tokens back
    for portions in ([300], [129, 1, 1, 2, 127, 40], [page - 1, 2, page, 1, 300 - 2 * page - 2]):
        got = run_mixer(part, x, portions, page_size=page)
        assert float((got.double() - want).abs().max()) < 2e-4, portions


@pytest.mark.parametrize("experts, top, ff", [(5, 2, 36), (3, 3, 24), (4, 1, 40), (33, 4, 17)])
def test_mixture_of_experts_alone(experts, top, ff):
    gen = torch.Generator().manual_seed(experts)
    w = 40
    t = {"f.router": draw(gen, (experts, w), 0.6), "f.router.b": draw(gen, (experts,), 0.3)}
    for e in range(experts):
        t.update({f"f.e{e}.gate": draw(gen, (ff, w), 0.2), f"f.e{e}.up": draw(gen, (ff, w), 0.2), f"f.e{e}.down": draw(gen, (w, ff), 0.2)})
    part = part_with_weights("ffn", PartSpec("moe", dict(hidden_size=w, expert_size=ff, experts=experts, top=top)), "f", torch.float32, t)
    x = draw(gen, (70, w))
    cfg = {"router": {"experts": experts, "top": top}}
    want = plain.routed_ff(x.double(), {k: v.double() for k, v in t.items()}, "f", cfg)
    harness = PartHarness({}, torch.float32)
    for n in (70, 1, 33):
        prepared = harness.prepare({f"r{n}": n})
        stream = ResidualStream(torch.zeros((n, w), dtype=torch.float32, device=DEV))
        stream.push(part.forward(prepared.ctx, x[:n].to(DEV).contiguous(), stream))
        stream.flush()
        assert float((stream.residual.cpu().double() - want[:n]).abs().max()) < 1e-4, n


def test_dense_feed_forward_and_offset_norm_alone():
    gen = torch.Generator().manual_seed(1)
    w, ff = 40, 100
    t = {"f.up": draw(gen, (ff, w), 0.4), "f.down": draw(gen, (w, ff), 0.2)}
    part = part_with_weights("ffn", PartSpec("gelu_mlp", dict(hidden_size=w, intermediate_size=ff)), "f", torch.float32, t)
    x = draw(gen, (19, w), 2.0)
    harness = PartHarness({}, torch.float32)
    prepared = harness.prepare({"a": 19})
    stream = ResidualStream(torch.zeros((19, w), dtype=torch.float32, device=DEV))
    stream.push(part.forward(prepared.ctx, x.to(DEV).contiguous(), stream))
    stream.flush()
    want = plain.dense_ff(x.double(), {k: v.double() for k, v in t.items()}, "f")
    assert float((stream.residual.cpu().double() - want).abs().max()) < 1e-4
    g = draw(gen, (w,), 0.3)
    norm = part_with_weights("norm", PartSpec("rmsnorm", {"size": w, "eps": 1e-3, "offset": 1.0, "weight_suffix": ""}), "n", torch.float32, {"n": g})
    stream = ResidualStream(x.to(DEV).contiguous())
    got = norm.forward(stream, harness.status)
    assert float((got.cpu().double() - plain.offset_norm(x.double(), g.double(), 1e-3)).abs().max()) < 1e-5


# ---- the tensor-core forms of the bfloat16 kernels against the CUDA-core forms ---------------------------

def bf16_mixer_both_ways(part, x, portions, toggle, page_size=16):
    outs = []
    for on in (True, False):
        toggle(on)
        try:
            outs.append(run_mixer(part, x, portions, page_size=page_size))
        finally:
            toggle(True)
    return outs


@pytest.mark.parametrize("heads, rank, rot", [(16, 64, 16), (20, 136, 8), (3, 512, 64)])
def test_latent_attention_on_tensor_cores(heads, rank, rot):
    from clockwork_b200.ops import latent as latent_ops

    gen = torch.Generator().manual_seed(heads)
    w, dim, vdim, q_rank = 64, 16, 24, 32
    t = {"m.dq": draw(gen, (q_rank, w), 0.3), "m.dq.norm": draw(gen, (q_rank,), 0.2, 1.0), "m.uq": draw(gen, (heads * (dim + rot), q_rank), 1.0),
         "m.dkv": draw(gen, (rank + rot, w), 0.6), "m.dkv.norm": draw(gen, (rank,), 0.2, 1.0), "m.uk": draw(gen, (heads * dim, rank), 0.3),
         "m.uv": draw(gen, (heads * vdim, rank), 0.2), "m.sink": draw(gen, (heads,), 1.5, 2.0), "m.g": draw(gen, (heads * vdim, w), 0.3),
         "m.o": draw(gen, (w, heads * vdim), 0.2)}
    cfg = dict(heads=heads, dim=dim, rot_dim=rot, vdim=vdim, kv_rank=rank, q_rank=q_rank, scale=0.35, rot={"base": 300.0, "dims": rot})
    spec = PartSpec("latent_attention", dict(hidden_size=w, heads=heads, dim=dim, rot_dim=rot, vdim=vdim, kv_rank=rank, q_rank=q_rank,
                                             scale=0.35, rope_base=300.0, eps=1e-5))
    part = part_with_weights("mixer", spec, "m", torch.bfloat16, t)
    x = draw(gen, (200, w))
    wd = {k: v.double() for k, v in t.items()}
    want = plain.latent_attention_mixer(x.double(), wd, "m", cfg, 1e-5)
    yard = float((plain.latent_attention_mixer(x.double(), wd, "m", cfg, 1e-5, rnd=plain.to_bfloat16_and_back) - want).abs().max())
    for portions in ([200], [63, 1, 1, 2, 64, 69]):
        fast, slow = bf16_mixer_both_ways(part, x, portions, latent_ops.set_tensor_cores)
        assert float((fast.double() - want).abs().max()) <= 3 * yard, portions
        assert float((slow.double() - want).abs().max()) <= 3 * yard, portions
        assert float((fast - slow).abs().max()) <= yard, portions


@pytest.mark.parametrize("experts, top, ff, w, n", [(7, 3, 136, 256, 300), (64, 6, 64, 128, 9), (5, 5, 40, 64, 130)])
def test_products_in_groups_on_tensor_cores(experts, top, ff, w, n):
    from clockwork_b200.ops import grouped as grouped_ops

    gen = torch.Generator().manual_seed(experts)
    t = {"f.router": draw(gen, (experts, w), 0.6), "f.router.b": draw(gen, (experts,), 0.3)}
    for e in range(experts):
        t.update({f"f.e{e}.gate": draw(gen, (ff, w), 0.2), f"f.e{e}.up": draw(gen, (ff, w), 0.2), f"f.e{e}.down": draw(gen, (w, ff), 0.2)})
    part = part_with_weights("ffn", PartSpec("moe", dict(hidden_size=w, expert_size=ff, experts=experts, top=top)), "f", torch.bfloat16, t)
    x = draw(gen, (n, w))
    cfg = {"router": {"experts": experts, "top": top}}
    wd = {k: v.double() for k, v in t.items()}
    want = plain.routed_ff(x.double(), wd, "f", cfg)
    yard = float((plain.routed_ff(x.double(), wd, "f", cfg, rnd=plain.to_bfloat16_and_back) - want).abs().max())
    harness = PartHarness({}, torch.bfloat16)
    outs = []
    for on in (True, False):
        grouped_ops.set_tensor_cores(on)
        try:
            prepared = harness.prepare({f"r{on}": n})
            stream = ResidualStream(torch.zeros((n, w), dtype=torch.float32, device=DEV))
            stream.push(part.forward(prepared.ctx, x.to(DEV, torch.bfloat16).contiguous(), stream))
            stream.flush()
            outs.append(stream.residual.cpu())
        finally:
            grouped_ops.set_tensor_cores(True)
    for got in outs:
        assert float((got.double() - want).abs().max()) <= 3 * yard
    assert float((outs[0] - outs[1]).abs().max()) <= yard


@pytest.mark.timeout(600)
def test_a_step_of_eight_layers_at_layer_sizes_of_published_models():
    """Eight layers at 2,048 width (grids of thousands of blocks, blocks with tens of kilobytes of shared memory, some
    300 launches a step): prompt portions and single-token steps through the captured graphs finish and agree with the
    same steps launched kernel by kernel."""
    from clockwork_b200.cache import CacheManager
    from clockwork_b200.cli import shape_config
    from clockwork_b200.engine import ModelRunner, StepEntry, random_model

    raw = shape_config("rapitar-2k")
    model = random_model(raw, seed=3, dtype="bfloat16", device=DEV)
    prompt = tokens_for({"vocab": raw["vocab"]}, 300, salt=9)
    tail = tokens_for({"vocab": raw["vocab"]}, 3, salt=10)
    results = []
    for graphs in (True, False):
        cache = CacheManager(model.cache_needs(), num_pages=64, page_size=16, dtype=model.dtype, device=DEV, num_state_slots=2)
        runner = ModelRunner(model, cache)
        if graphs:
            assert runner.enable_graphs(max_ctx=1024, max_batch=2)
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
        assert not graphs or (runner.portion_graph_steps == 1 and runner.graphs)
        results.append(torch.cat(rows))
    assert torch.isfinite(results[0]).all()
    scale = float(results[1].abs().max())
    assert float((results[0] - results[1]).abs().max()) <= 0.02 * scale
