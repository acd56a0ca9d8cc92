"""The Giforax design on the GPU against the plain implementation (tests/plain_giforax.py): each mechanism alone, the
residual stream layer by layer, whole prompts, token-by-token decoding, portions down to two tokens, mixed batches on
a tight pool with four slots, long decoding, keys at the edges of chunks and pages, slots and pages used again, greedy
generation through the engine's entry point, and the trace program."""
import json

import numpy as np
import pytest
import torch

import plain_giforax
import replay_util
from giforax_configs import CONFIGS, attention, moe
from gpu_common import F32_ATOL, F32_RTOL, need_gpu, note_worst

pytestmark = pytest.mark.gpu
CUDA = torch.device("cuda")
# float32: every row is compared, with the bounds the Llama tests use.  A router whose last chosen score lies within
# CLOSE (as a share of itself) of the next one may choose otherwise after rounding, which is no rounding error: such a
# token's own row is left out.
# bfloat16: rows kept in bfloat16 between kernels move a router's scores, so now and then a token is routed otherwise
# than in the float64 model, and what it then leaves in keys and state is read by later tokens.  The bound there is
# statistical: nine rows in ten within BF16_REL of the sequence's largest logit, the median within a third of it.
CLOSE = {"float32": 1e-5, "bfloat16": 0.1}
BF16_REL = 0.03


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    from torchinferno_b200.weights.random_init import write_random_model
    return {name: write_random_model(config, tmp_path_factory.mktemp(name), seed) for name, (config, seed) in CONFIGS.items()}


_plain: dict = {}


def plain(folder, tokens, dtype):
    """(logits [T, vocab], positions that a router's close call makes incomparable)."""
    key = (str(folder), tuple(tokens))
    if key not in _plain:
        if str(folder) not in _plain:
            _plain[str(folder)] = plain_giforax.read_model_folder(folder)
        config, weights = _plain[str(folder)]
        gaps = [[] for _ in tokens]
        _plain[key] = (plain_giforax.forward(config, weights, tokens, gaps=gaps).numpy(), [min(g, default=1.0) for g in gaps])
    logits, gaps = _plain[key]
    return logits, {t for t, g in enumerate(gaps) if g < CLOSE[dtype]}


def requests_for(config, seed, lengths):
    g = torch.Generator().manual_seed(700 + seed)
    return {f"q{i}": torch.randint(0, config["vocab"], (n,), generator=g).tolist() for i, n in enumerate(lengths)}


def compare(rows, folder, requests, dtype, what):
    shares = []
    for (name, pos), got_list in rows.items():
        ref, close = plain(folder, requests[name], dtype)
        if pos in close:
            continue
        for got in got_list:
            got = np.asarray(got, dtype=np.float64)
            assert np.isfinite(got).all(), f"{name}@{pos}: non-finite logits"
            err = np.abs(got - ref[pos]).max()
            if dtype == "float32":
                bound = F32_ATOL + F32_RTOL * np.abs(ref[pos]).max()
                assert err <= bound, f"{what}: {name}@{pos} ({dtype}): max error {err:.3e} exceeds {bound:.3e}"
            else:
                bound = BF16_REL * np.abs(ref).max()
            shares.append(err / bound)
    assert len(shares) >= max(1, len(rows) // 6), f"{what}: only {len(shares)} of {len(rows)} rows could be compared"
    shares = np.sort(np.asarray(shares))
    if dtype == "float32":
        note_worst(f"giforax {what} [{dtype}]", shares[-1])
    else:
        ninth, median = shares[int(0.9 * (len(shares) - 1))], shares[len(shares) // 2]
        assert ninth <= 1.0 and median <= 1 / 3, f"{what} ({dtype}): nine in ten rows within {ninth:.2f} of the bound, median {median:.2f}"
        note_worst(f"giforax {what}, nine rows in ten [{dtype}]", ninth)


def make_runner(folder, dtype, max_tokens, page_size=16, max_requests=4):
    from torchinferno_b200.engine.factory import load_model, make_runner as make
    model = load_model(folder, dtype=dtype)
    return make(model, page_size=page_size, max_tokens=max_tokens + page_size * max_requests, max_requests=max_requests)


def run_steps(runner, steps):
    from torchinferno_b200.engine.batch import StepEntry
    out = {}
    with torch.inference_mode():
        for step in steps:
            logits = runner.step([StepEntry(e["id"], e["tokens"], e["want"]) for e in step["entries"]])
            if logits.shape[0]:
                out[step["step"]] = logits.cpu().numpy()
            runner.end(step["end"])
            runner.cache.audit()
    return out


# ------------------------------------------------------------ whole models
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_the_residual_stream_after_every_layer(name, folders):
    need_gpu()
    from torchinferno_b200.engine.batch import StepEntry
    from torchinferno_b200.parts.sandwich_block import SandwichBlock
    config, seed = CONFIGS[name]
    tokens = requests_for(config, seed, [45])["q0"]
    cfg, w = plain_giforax.read_model_folder(folders[name])
    _, want = plain_giforax.forward(cfg, w, tokens, return_layers=True)
    runner = make_runner(folders[name], "float32", 64)
    seen, original = [], SandwichBlock.forward

    def recording(self, stream, ctx):
        original(self, stream, ctx)
        seen.append(stream.residual.clone())
    SandwichBlock.forward = recording
    try:
        with torch.inference_mode():
            runner.step([StepEntry("a", tokens, [0])])
    finally:
        SandwichBlock.forward = original
    assert len(seen) == want.shape[0]
    for i, got in enumerate(seen):
        err = (got.cpu().double() - want[i]).abs().max()
        assert err <= 1e-4 * want[i].abs().max(), f"layer {i}: {err:.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_whole_tail_portions_and_mixed_batches(name, dtype, folders):
    need_gpu()
    config, seed = CONFIGS[name]
    requests = requests_for(config, seed, [1, 2, 37, 70, 131, 64, 33])
    page = {"GA": 16, "GB": 4, "GC": 8, "GD": 8, "GE": 2}[name]
    for kind, (steps, index) in {
            "whole": replay_util.trace_whole(requests), "tail": replay_util.trace_tail_decode(requests, tail=40),
            "portions": replay_util.trace_portions(requests, sizes=(2, 7, 16, 3, 33, 2, 5, 31, 32, 2, 64)),
            "mixed": replay_util.trace_mixed(requests, seed=seed)}.items():
        runner = make_runner(folders[name], dtype, replay_util.peak_tokens(steps), page_size=page)
        rows = replay_util.gather(run_steps(runner, steps), index)
        compare(rows, folders[name], requests, dtype, f"{name} {kind}")
        assert not runner.cache.live_requests


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_every_token_decoded_alone_from_the_first_and_long_decoding(dtype, folders):
    need_gpu()
    config, seed = CONFIGS["GA"]
    requests = requests_for(config, seed + 5, [150, 9])
    steps, index = replay_util.trace_tail_decode(requests, tail=10 ** 6)       # one token a step from position 0
    runner = make_runner(folders["GA"], dtype, replay_util.peak_tokens(steps), page_size=4)
    rows = replay_util.gather(run_steps(runner, steps), index)
    assert runner.counters["graph_steps"] > 100                              # the captured decode pass ran them
    compare(rows, folders["GA"], requests, dtype, "GA token by token")


def test_a_batch_of_unequal_requests_gives_each_what_it_gets_alone(folders):
    need_gpu()
    from torchinferno_b200.engine.batch import StepEntry
    config, seed = CONFIGS["GA"]
    reqs = requests_for(config, seed + 9, [150, 3, 69, 1])
    runner = make_runner(folders["GA"], "float32", 4 * 192, page_size=8)
    with torch.inference_mode():
        alone = {}
        for k, toks in reqs.items():
            alone[k] = runner.step([StepEntry(k + "a", toks, list(range(len(toks))))]).cpu()
            runner.end([k + "a"])
        # together: a portion of each, then the rest of each, in another order (slots and pages are used again)
        first = {k: max(1, len(t) // 2) for k, t in reqs.items()}
        got = {k: [] for k in reqs}
        out = runner.step([StepEntry(k, reqs[k][:first[k]], list(range(first[k]))) for k in reqs]).cpu()
        row = 0
        for k in reqs:
            got[k].append(out[row:row + first[k]]); row += first[k]
        rest = [k for k in reversed(list(reqs)) if len(reqs[k]) > first[k]]
        out = runner.step([StepEntry(k, reqs[k][first[k]:], list(range(len(reqs[k]) - first[k]))) for k in rest]).cpu()
        row = 0
        for k in rest:
            n = len(reqs[k]) - first[k]
            got[k].append(out[row:row + n]); row += n
        runner.end(list(reqs))
    for k in reqs:
        assert torch.allclose(torch.cat(got[k]), alone[k], atol=2e-6, rtol=2e-5), k


# ------------------------------------------------------- mechanisms alone
def _entries_batch(entries):
    from torchinferno_b200.engine.batch import EntryPlacement, build_batch
    places, row = [], 0
    for rid, slot, start, n in entries:
        places.append(EntryPlacement(rid, slot, row, n, start))
        row += n
    batch, _ = build_batch(places, [[0] * p.q_len for p in places], [[] for _ in places], [], CUDA)
    return batch


def _random_weights(part, seed, dtype, prefix):
    """Bind seeded random weights (stored in bfloat16, as a checkpoint would) and return them in float64 by full name."""
    from torchinferno_b200.weights.random_init import random_tensor
    stored = {ws.name: random_tensor(ws, seed, dtype=torch.bfloat16) for ws in part.weight_specs()}
    vectors = {ws.name for ws in part.weight_specs() if ws.role == "vector"}
    part.bind({k: (v.float() if dtype == torch.float32 or k in vectors else v).cuda() for k, v in stored.items()})
    return {prefix + k: v.double() for k, v in stored.items()}


def _apply_tables(cache):
    from torchinferno_b200.kernels import ops
    for group, (idx, val) in zip(cache.groups, cache.drain_table_updates()):
        if idx:
            ops.scatter_i32(group.table_device, torch.tensor(idx, dtype=torch.int32).cuda(), torch.tensor(val, dtype=torch.int32).cuda())


def _kv_context(cache, entries, writes=True):
    from torchinferno_b200.parts.base import KVBinding, LayerContext
    b = cache.kv_binding(0)
    return LayerContext(batch=_entries_batch(entries), error_word=cache.error_word,
                        kv=KVBinding(b.pool, b.block_table, b.page_size, b.window, writes, b.keys, b.values))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,size,page", [(4, 2, 16, 24, 20, 8), (3, 1, 40, 8, 7, 4), (2, 2, 64, 64, 64, 16)])
def test_sigmoid_attention_alone_at_the_edges_of_chunks_and_pages(dtype, heads, kv_heads, dim, vdim, size, page):
    """A prompt in portions, then single tokens, in a pool whose pages were used before.  The first token of every
    chunk and the last token of the chunk before it carry values thirty times the usual size: a query that reads one key
    too many or one too few, on either side of a chunk's edge, in a prompt or decoded alone, is far off; so is one
    that reads a wrong page."""
    need_gpu()
    from torchinferno_b200.cache.manager import CacheManager
    from torchinferno_b200.parts.base import PartSpec, build_part
    W, eps = 48, 1e-5
    m = attention(heads, kv_heads, dim, vdim, size, 0.3, rot_dims=dim // 2 if dim % 4 == 0 else dim, base=1000.0)
    params = {"hidden_size": W, "heads": heads, "kv_heads": kv_heads, "dim": dim, "value_dim": vdim, "scale": 0.3,
              "position": PartSpec("rotary", {"head_dim": dim, "theta": 1000.0, "rot_dim": m["rot"]["dims"]}),
              "qk_norm_eps": eps, "chunk": size}
    mixer = build_part("mixer", PartSpec("sigmoid_attention", params), dtype=dtype, device=CUDA)
    w = _random_weights(mixer, 3, dtype, "mix.")
    T = 3 * size + 5 + 14
    g = torch.Generator().manual_seed(size)
    x = torch.randn(T, W, generator=g)
    for c in range(1, 4):
        x[c * size] *= 30
        x[c * size - 1] *= 30
    x = x.to(dtype)
    pos = torch.arange(T)
    keys, values = plain_giforax.attention_keys_values(x.double(), w, "mix.", m, eps, pos)
    want = plain_giforax.attention_mixer(x.double(), w, "mix.", m, eps, pos, keys, values)
    # what a mask one key off would give, at the second query of the last whole chunk
    q_edge = 3 * size
    lost = values.clone(); lost[q_edge] = 0          # the chunk's own first key left out
    leaked = plain_giforax.attention_mixer(x.double()[q_edge - 1:], w, "mix.", dict(m, mask={"size": 10 ** 6}), eps, pos[q_edge - 1:],
                                           keys[q_edge - 1:], values[q_edge - 1:])     # the key before the edge let in
    assert (plain_giforax.attention_mixer(x.double(), w, "mix.", m, eps, pos, keys, lost)[q_edge + 1] - want[q_edge + 1]).abs().max() \
        > 0.2 * want[q_edge + 1].abs().max()
    assert (leaked[2] - want[q_edge + 1]).abs().max() > 0.05 * want[q_edge + 1].abs().max()
    pages = -(-T // page) + 4
    cache = CacheManager([mixer.cache_spec()], [None], page_size=page, num_pages=pages, max_requests=3, max_request_tokens=T + page,
                         dtype=dtype, device=CUDA)
    cache.groups[0].pool.fill_(float("nan"))
    cache.open("old"), cache.extend("old", 2 * page + 1), cache.open("warm"), cache.extend("warm", page + 1)
    cache.close("old")                  # its pages go to "r", out of order
    cache.open("r")
    outs, at = [], 0
    portions = [size - 1, 2, size - 1, 1, 1, size + 3]
    portions += [1] * (T - sum(portions))
    for n in portions:
        start = cache.extend("r", n)
        _apply_tables(cache)
        outs.append(mixer.forward(x[at:at + n].cuda().contiguous(), _kv_context(cache, [("r", cache.slot("r"), start, n)])))
        at += n
    assert at == T and int(cache.error_word) == 0
    got = torch.cat(outs).cpu().double()
    tol = 2e-5 if dtype == torch.float32 else BF16_REL
    err = (got - want).abs().max(dim=1).values / want.abs().max()
    assert err.max() <= tol, (int(err.argmax()), float(err.max()))
    # a layer without keys of its own reads the same cache with its own queries and mask
    reader = build_part("mixer", PartSpec("sigmoid_attention", dict(params, own_kv=False, chunk=size + 3)), dtype=dtype, device=CUDA)
    w2 = _random_weights(reader, 4, dtype, "mix.")
    y = torch.randn(T, W, generator=g).to(dtype)
    want2 = plain_giforax.attention_mixer(y.double(), w2, "mix.", dict(m, mask={"size": size + 3}), eps, pos, keys, values)
    out = torch.cat([reader.forward(y[a:b].cuda().contiguous(), _kv_context(cache, [("r", cache.slot("r"), a, b - a)], writes=False))
                     for a, b in ((0, size + 2), (size + 2, size + 3), (size + 3, T))]).cpu().double()
    if dtype == torch.bfloat16:     # (the oracle's keys are exact, the cache's are rounded to bfloat16)
        want2 = plain_giforax.attention_mixer(y.double(), w2, "mix.", dict(m, mask={"size": size + 3}), eps, pos,
                                              keys.to(dtype).double(), values.to(dtype).double())
    assert ((out - want2).abs().max() / want2.abs().max()) <= tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_sigmoid_attention_finds_a_far_key_among_hundreds(dtype):
    """One long chunk: 700 keys over pages of 16, the key at position 3 with a value a hundred times the usual size and a
    score made large for the last queries.  Decoded tokens and a prompt's tail must both see it."""
    need_gpu()
    from torchinferno_b200.cache.manager import CacheManager
    from torchinferno_b200.parts.base import PartSpec, build_part
    W, eps, T, far = 32, 1e-6, 700, 3
    m = attention(2, 1, 16, 16, 4096, 1.0, rot_dims=4, base=100.0)
    mixer = build_part("mixer", PartSpec("sigmoid_attention", {
        "hidden_size": W, "heads": 2, "kv_heads": 1, "dim": 16, "value_dim": 16, "scale": 1.0, "qk_norm_eps": eps, "chunk": 4096,
        "position": PartSpec("rotary", {"head_dim": 16, "theta": 100.0, "rot_dim": 4})}), dtype=dtype, device=CUDA)
    w = _random_weights(mixer, 9, dtype, "mix.")
    x = torch.randn(T, W, generator=torch.Generator().manual_seed(1)) * 0.3
    x[far] *= 100
    x = x.to(dtype)
    pos = torch.arange(T)
    keys, values = plain_giforax.attention_keys_values(x.double(), w, "mix.", m, eps, pos)
    want = plain_giforax.attention_mixer(x.double(), w, "mix.", m, eps, pos, keys, values)
    lost = values.clone(); lost[far] = 0
    without = plain_giforax.attention_mixer(x.double(), w, "mix.", m, eps, pos, keys, lost)
    assert (without[-1] - want[-1]).abs().max() > 0.3 * want[-1].abs().max()
    cache = CacheManager([mixer.cache_spec()], [None], page_size=16, num_pages=48, max_requests=2, max_request_tokens=720,
                         dtype=dtype, device=CUDA)
    cache.open("r")
    outs, at = [], 0
    for n in [2, 300, 390] + [1] * 8:
        start = cache.extend("r", n)
        _apply_tables(cache)
        outs.append(mixer.forward(x[at:at + n].cuda().contiguous(), _kv_context(cache, [("r", cache.slot("r"), start, n)])))
        at += n
    got = torch.cat(outs).cpu().double()
    tol = 2e-5 if dtype == torch.float32 else BF16_REL
    assert (got - want).abs().max() <= tol * want.abs().max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [72, 20, 256])
def test_minimal_gru_alone_in_portions_over_its_state(dtype, width):
    """Portions that end just before, at and just after the kernel's run of 64 tokens, long ones that are scanned run by
    run, single tokens; a first token that must still show at the end (its gate is opened wide and every later gate
    nearly shut); two requests in one step; a slot used again starts from zero."""
    need_gpu()
    from torchinferno_b200.cache.manager import CacheManager
    from torchinferno_b200.parts.base import LayerContext, PartSpec, build_part
    W = 48
    mixer = build_part("mixer", PartSpec("min_gru", {"hidden_size": W, "width": width}), dtype=dtype, device=CUDA)
    w = _random_weights(mixer, 4, dtype, "mix.")
    g = torch.Generator().manual_seed(width)
    T = 63 + 1 + 2 + 64 + 65 + 1 + 200 + 1 + 1 + 130
    x = torch.randn(T, W, generator=g).to(dtype)
    other = torch.randn(80, W, generator=g).to(dtype)
    m = {"width": width}
    want, _ = plain_giforax.min_gru_mixer(x.double(), w, "mix.", m)
    want_other, _ = plain_giforax.min_gru_mixer(other.double(), w, "mix.", m)
    # the state a request leaves is what the next portion starts from: the last portion from a zero state differs
    assert (plain_giforax.min_gru_mixer(x.double()[T - 130:], w, "mix.", m)[0][0] - want[T - 130]).abs().max() > 0.05 * want[T - 130].abs().max()
    cache = CacheManager([], [mixer.state_spec()], page_size=4, num_pages=4, max_requests=2, max_request_tokens=10 ** 6,
                         dtype=dtype, device=CUDA)
    cache.open("warm"), cache.close("warm")
    slot_r, slot_o = cache.open("r"), cache.open("o")
    outs, outs_other, pos, opos = [], [], 0, 0
    for n, k in ((63, 0), (1, 7), (2, 0), (64, 1), (65, 0), (1, 64), (200, 0), (1, 0), (1, 8), (130, 0)):
        entries = [("r", slot_r, pos, n)] + ([("o", slot_o, opos, k)] if k else [])
        rows = torch.cat([x[pos:pos + n]] + ([other[opos:opos + k]] if k else [])).cuda().contiguous()
        out = mixer.forward(rows, LayerContext(batch=_entries_batch(entries), state=cache.states[0]))
        outs.append(out[:n]), outs_other.append(out[n:])
        pos, opos = pos + n, opos + k
    assert pos == T
    got, got_other = torch.cat(outs).cpu().double(), torch.cat(outs_other).cpu().double()
    tol = 2e-5 if dtype == torch.float32 else BF16_REL
    assert (got - want).abs().max() <= tol * want.abs().max()
    assert (got_other - want_other[:opos]).abs().max() <= tol * want_other.abs().max()
    cache.close("o")
    assert cache.open("n") == slot_o
    out = mixer.forward(other[:5].cuda().contiguous(), LayerContext(batch=_entries_batch([("n", slot_o, 0, 5)]), state=cache.states[0]))
    assert (out.cpu().double() - want_other[:5]).abs().max() <= tol * want_other.abs().max()


def test_minimal_gru_keeps_a_first_token_through_a_long_quiet_run():
    """Gates made by hand: wide open at the first token, shut (z about 1e-4) at the 500 that follow, in portions and
    single tokens.  A state that is reset, scaled or lost at a run's or a portion's edge shows in the last outputs."""
    need_gpu()
    from torchinferno_b200.kernels import ops
    width, T = 40, 501
    proj = torch.zeros(T, 3 * width)
    proj[0, :width] = 9.0                                   # z = sigmoid(9)
    proj[1:, :width] = -9.0
    proj[:, width:2 * width] = torch.linspace(-2, 2, width)[None] + 0.01 * torch.randn(T, width)
    proj[:, 2 * width:] = 1.0
    z = torch.sigmoid(proj[:, :width].double())
    u = proj[:, width:2 * width].double()
    c = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    S, want = torch.zeros(width, dtype=torch.float64), []
    for t in range(T):
        S = (1 - z[t]) * S + z[t] * c[t]
        want.append(S * (1.0 / (1 + np.exp(-1.0))))
    want = torch.stack(want)
    assert (want[-1] / want[0]).min() > 0.9                 # the first token is nearly all there is at the end
    state = torch.zeros(2, width, device=CUDA)
    state[0] = 5.0                                          # (another slot's state must not leak)
    out = torch.empty(T, width, device=CUDA)
    at = 0
    for n in (1, 63, 64, 129, 1, 1, 242):
        q_start = torch.tensor([0, n], dtype=torch.int32, device=CUDA)
        ops.gated_recurrence(proj[at:at + n].cuda().contiguous(), 0, width, 2 * width, None, None, state, q_start,
                             torch.tensor([1], dtype=torch.int32, device=CUDA), out[at:at + n], 1, n)
        at += n
    assert at == T and (out.cpu().double() - want).abs().max() <= 1e-4 * want.abs().max()
    assert float((state[0] - 5.0).abs().max()) == 0.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts,top,shared,tokens", [(5, 2, 24, 300), (3, 3, 0, 70), (9, 1, 16, 3), (40, 4, 0, 200)])
def test_routed_gated_units_alone(dtype, experts, top, shared, tokens):
    need_gpu()
    from torchinferno_b200.parts.base import LayerContext, PartSpec, build_part
    W, ff = 40, 24
    part = build_part("feed_forward", PartSpec("routed_experts", {
        "hidden_size": W, "experts": experts, "top": top, "expert_size": ff, "activation": "glu_clamp", "limit": 0.8,
        "shared_limit": 1.7, "scores": "sigmoid", "normalize": False, "weight_on_input": True, "shared_size": shared}),
        dtype=dtype, device=CUDA)
    w = _random_weights(part, experts, dtype, "mlp.")
    x = (torch.randn(tokens, W, generator=torch.Generator().manual_seed(tokens)) * 1.5).to(dtype)
    mlp = moe(experts, top, ff, 0.8, shared or None, 1.7)
    gaps = [[] for _ in range(tokens)]
    want = plain_giforax.routed_feed_forward(x.double(), w, "mlp.", mlp, gaps)
    # the clamps bite, and the weight sits on the input (on the output it would give something else)
    pre = x.double() @ w["mlp.e0.gate"].T
    assert (pre > 0.8).any() and (x.double() @ w["mlp.e0.up"].T < -0.8).any()
    got = part.forward(x.cuda().contiguous(), LayerContext(batch=None)).cpu().double()
    # (the router reads the same rows in both number formats, in 32-bit: only a tie within its rounding is unclear)
    clear = torch.tensor([min(gp, default=1.0) >= 1e-5 for gp in gaps])
    assert clear.sum() >= tokens // 3
    tol = 2e-5 if dtype == torch.float32 else BF16_REL
    assert (got - want)[clear].abs().max() <= tol * want.abs().max()
    if top < experts:       # the tokens really go to different experts
        assert len(set(torch.sigmoid(x.double() @ w["mlp.router"].T).argmax(-1).tolist())) > 1


@pytest.mark.parametrize("width,rows", [(44, 7), (50, 9), (192, 300), (4096, 5), (9000, 3)])
def test_layer_norm_and_the_tails_of_sublayers(width, rows):
    """The norm alone (gathered rows too), and the fused tail: norm of a sublayer's output, sum into the residual, the
    average over the layers so far, the norm that opens what follows.  Rows with a large mean, where a one-pass variance
    would lose digits."""
    need_gpu()
    from torchinferno_b200.kernels import ops
    g = torch.Generator().manual_seed(width)
    eps = 1e-5

    def ln(x, wt, b):
        mean = x.mean(-1, keepdim=True)
        return (x - mean) / torch.sqrt((x - mean).pow(2).mean(-1, keepdim=True) + eps) * wt + b

    wa, ba, wb, bb = (torch.randn(width, generator=g) for _ in range(4))
    x = torch.randn(rows, width, generator=g) + 300.0
    pick = torch.tensor([rows - 1, 0, rows // 2], dtype=torch.int32)
    out = ops.layernorm(x.cuda(), wa.cuda(), ba.cuda(), eps, torch.empty(3, width, device=CUDA), pick.cuda())
    assert (out.cpu().double() - ln(x.double(), wa.double(), ba.double())[pick.long()]).abs().max() <= 3e-4
    for dtype in (torch.float32, torch.bfloat16):
        count = 4
        history = torch.randn(count + 1, rows, width, generator=g)
        y = (torch.randn(rows, width, generator=g) * 3 + 2).to(dtype)
        coef = torch.randn(count, generator=g)
        want_res = history[count - 1].double() + ln(y.double(), wa.double(), ba.double())
        want_next = sum(coef[j].double() * (history[j].double() if j < count - 1 else want_res) for j in range(count))
        want_out = ln(want_next, wb.double(), bb.double())
        h = history.cuda()
        normed = torch.empty(rows, width, dtype=dtype, device=CUDA)
        ops.layernorm_tail(h[count - 1], eps, y=y.cuda(), y_norm=(wa.cuda(), ba.cuda()), history=h, coef=coef.cuda(), count=count,
                           out=normed, out_norm=(wb.cuda(), bb.cuda()))
        assert (h[count - 1].cpu().double() - want_res).abs().max() <= 2e-5 * want_res.abs().max()
        assert (h[count].cpu().double() - want_next).abs().max() <= 2e-5 * want_next.abs().max()
        assert (h[:count - 1].cpu() == history[:count - 1]).all()
        tol = 2e-4 if dtype == torch.float32 else 0.02
        assert (normed.cpu().double() - want_out).abs().max() <= tol * want_out.abs().max()


# ------------------------------------------------- the two attention kernels
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,chunk,page", [(6, 2, 64, 64, 200, 16), (16, 8, 128, 128, 512, 16), (3, 1, 40, 24, 7, 8),
                                                             (4, 4, 72, 128, 64, 32), (5, 1, 16, 8, 0, 4), (70, 1, 32, 32, 129, 16)])
def test_sigmoid_attention_kernels_agree_with_plain_arithmetic(heads, kv_heads, dim, vdim, chunk, page):
    """The tensor-core kernel and the CUDA-core kernel on the same bf16 pages, against float64: a ragged step (prompt
    portions that begin and end off the 64-key tile edges and the chunk edges, beside single tokens) and a step of single
    tokens with contexts just below, at and above tile, page and chunk edges.  Unwritten cache holds NaN."""
    need_gpu()
    from torchinferno_b200.kernels import ops
    g = torch.Generator().manual_seed(heads * dim + chunk)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=CUDA)
    c = chunk or 10 ** 6
    cases = {"ragged": [(0, 70), (63, 2), (64, 1), (100, 129), (5, 1), (c - 1 if chunk else 30, 3)],
             "single": [(0, 1), (62, 1), (63, 1), (64, 1), (127, 1), (300, 1), (c - 1 if chunk else 511, 1), (c if chunk else 512, 1), (2 * c + 1 if chunk else 77, 1)]}
    group = heads // kv_heads
    for name, entries in cases.items():
        entries = [(s, n) for s, n in entries if s + n <= 1200]
        pages_per = max(-(-(start + n) // page) for start, n in entries)
        total = len(entries) * pages_per
        keys = torch.full((total, kv_heads, page, dim), float("nan")).to(torch.bfloat16)
        values = torch.full((total, kv_heads, page, vdim), float("nan")).to(torch.bfloat16)
        table = torch.randperm(total, generator=g).to(torch.int32).view(len(entries), pages_per)
        n_tokens = sum(n for _, n in entries)
        q = torch.randn(n_tokens, heads, dim, generator=g).to(torch.bfloat16)
        gate = torch.randn(n_tokens, heads + 3, generator=g).to(torch.bfloat16)
        bias = torch.randn(heads, generator=g)
        q_start = [0]
        for _, n in entries:
            q_start.append(q_start[-1] + n)
        want = torch.empty(n_tokens, heads, vdim, dtype=torch.float64)
        for e, (start, n) in enumerate(entries):
            ctx = start + n
            pos = torch.arange(ctx)
            krows = torch.randn(ctx, kv_heads, dim, generator=g).to(torch.bfloat16)
            vrows = torch.randn(ctx, kv_heads, vdim, generator=g).to(torch.bfloat16)
            keys[table[e][pos // page].long(), :, pos % page] = krows
            values[table[e][pos // page].long(), :, pos % page] = vrows
            qpos = start + torch.arange(n)
            seen = (pos[None, :] <= qpos[:, None]) & ((pos[None, :] // c) == (qpos[:, None] // c))
            qe = q[q_start[e]:q_start[e + 1]].double()
            for h in range(heads):
                score = qe[:, h] @ krows[:, h // group].double().T * 0.11 + bias[h].double()
                weight = torch.sigmoid(score) * seen
                want[q_start[e]:q_start[e + 1], h] = (weight @ vrows[:, h // group].double()) \
                    * torch.sigmoid(gate[q_start[e]:q_start[e + 1], h].double())[:, None]
        pool = torch.cat([keys.flatten(1), values.flatten(1)], dim=1).cuda().contiguous()
        kview = pool[:, :kv_heads * page * dim].unflatten(1, (kv_heads, page, dim))
        vview = pool[:, kv_heads * page * dim:].unflatten(1, (kv_heads, page, vdim))
        # (single tokens on the tensor cores: also with the keys of a context shared out over 1, 3 and 7 blocks)
        for simt, splits in ((False, None), (True, None)) + (((False, 1), (False, 3), (False, 7)) if name == "single" else ()):
            out = torch.empty(n_tokens, heads * vdim, dtype=torch.bfloat16, device=CUDA)
            ops.sigmoid_attention(q.view(n_tokens, heads * dim).cuda(), kview, vview, out, i32(q_start), i32([s for s, _ in entries]),
                                  i32(list(range(len(entries)))), table.cuda().contiguous(), len(entries), max(n for _, n in entries),
                                  heads, kv_heads, scale=0.11, chunk=chunk, head_bias=bias.cuda(), gate=gate.cuda()[:, :heads],
                                  force_simt=simt, max_kv_len=max(s + n for s, n in entries), splits=splits)
            got = out.view(n_tokens, heads, vdim).cpu().double()
            assert torch.isfinite(got).all(), f"{name}, simt={simt}, splits={splits}"
            err = (got - want).abs().max()
            assert err <= 6e-3 * want.abs().max(), f"{name}, simt={simt}, splits={splits}: {err:.3e} of {want.abs().max():.3e}"


# ------------------------------------------------ entry point and programs
def test_greedy_generation_through_the_engine_and_its_scheduler(folders):
    need_gpu()
    from torchinferno_b200.config.engine_config import EngineConfig
    from torchinferno_b200.engine.engine import InferenceEngine
    from torchinferno_b200.engine.types import GenerateRequest, SamplingConfig
    config, seed = CONFIGS["GA"]
    cfg, w = plain_giforax.read_model_folder(folders["GA"])
    prompts = list(requests_for(config, seed + 2, [5, 41, 1, 18, 66]).values())
    new = 12
    for dtype in ("float32", "bfloat16"):
        with InferenceEngine.from_config(EngineConfig(model=str(folders["GA"]), dtype=dtype, page_size=8, max_batch_size=3,
                                                      prefill_chunk_size=16, max_num_batched_tokens=48, kv_cache_tokens=512)) as engine:
            outs = engine.generate_many([GenerateRequest(f"g{i}", prompt_token_ids=p, sampling=SamplingConfig(new))
                                         for i, p in enumerate(prompts)])
        for prompt, out in zip(prompts, outs):
            tokens = list(out.token_ids)
            assert len(tokens) == new
            logits = plain_giforax.forward(cfg, w, (prompt + tokens)[:-1])
            for i, tok in enumerate(tokens):
                row = logits[len(prompt) + i - 1]
                best = row.topk(2)
                if dtype == "float32" and float(best.values[0] - best.values[1]) > 1e-4 * float(row.abs().max()):
                    assert tok == int(best.indices[0])
                else:
                    assert tok in best.indices.tolist()


def test_the_trace_program_replays_a_giforax_folder(folders, tmp_path):
    need_gpu()
    import subprocess
    import sys
    config, seed = CONFIGS["GB"]
    requests = requests_for(config, seed + 3, [30, 75, 2])
    steps, index = replay_util.trace_mixed(requests, seed=3)
    out_dir = tmp_path / "out"
    cmd = [sys.executable, str(replay_util.ROOT / "bin" / "trace_run"), "--model", str(folders["GB"]), "--dtype", "float32",
           "--out", str(out_dir), "--max-tokens", str(replay_util.peak_tokens(steps))]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    try:
        for step in steps:
            proc.stdin.write(json.dumps(step) + "\n")
            proc.stdin.flush()
            assert proc.stdout.readline().strip() == f"done {step['step']}"
        proc.stdin.close()
        assert proc.wait(timeout=120) == 0
    finally:
        if proc.poll() is None:
            proc.kill()
    results = {}
    for step in steps:
        wanted = sum(len(e["want"]) for e in step["entries"])
        if wanted:
            results[step["step"]] = np.fromfile(out_dir / f"{step['step']}.f32", dtype="<f4").reshape(wanted, config["vocab"])
    compare(replay_util.gather(results, index), folders["GB"], requests, "float32", "GB trace program")


# ------------------------------------------------------- sizes drawn at random
def _random_config(rng):
    """A small Giforax configuration with sizes drawn from lists that mix multiples of 8, 16, 64 with odd ones."""
    pick = rng.choice
    width = pick([24, 40, 72, 96, 136])
    layers, with_keys = [], []
    for i in range(pick([2, 3, 4])):
        form = pick(["moe", "moe", None])
        experts = pick([2, 4, 7])
        mlp = None if form is None else moe(experts, rng.randint(1, experts), pick([8, 24, 36]), pick([0.5, 2.0, 7.0]),
                                            shared=pick([None, 16, 28]), shared_limit=pick([1.0, 3.0]))
        if rng.random() < 0.3:
            layers.append({"type": "mingru", "mixer": {"width": pick([8, 33, 64, 100])}, "mlp": mlp})
            continue
        if with_keys and rng.random() < 0.5:
            source = pick(with_keys)
            sm = layers[source]["mixer"]
            group = pick([1, 2, 3])
            mixer = attention(sm["kv_heads"] * group, sm["kv_heads"], sm["dim"], sm["vdim"], pick([1, 3, 16, 50, 4096]),
                              pick([0.1, 0.3]), sm["rot"]["dims"], base=sm["rot"]["base"], kv_from=source)
        else:
            kv_heads, dim = pick([1, 2, 3]), pick([4, 8, 24, 40])
            mixer = attention(kv_heads * pick([1, 2, 4]), kv_heads, dim, pick([6, 8, 20, 40]), pick([1, 3, 16, 50, 4096]),
                              pick([0.1, 0.3]), pick([2, dim // 2, dim]) // 2 * 2 or 2, base=pick([100.0, 10000.0]))
            with_keys.append(i)
        layers.append({"type": "attention", "mixer": mixer, "mlp": mlp})
    return {"architecture": "Giforax", "vocab": pick([50, 97, 128]), "width": width, "norm": {"eps": pick([1e-6, 1e-5])},
            "embedding": {"scale": pick([0.5, 1.0, 12.0])}, "layers": layers}


@pytest.mark.parametrize("draw", range(8))
def test_sizes_drawn_at_random(draw, tmp_path):
    """Whole prompts, portions and token-by-token decoding of models whose every size was drawn at random, in both
    number formats (float32 row by row, bfloat16 by the statistical bound)."""
    need_gpu()
    import random
    from torchinferno_b200.weights.random_init import write_random_model
    rng = random.Random(5200 + draw)
    config = _random_config(rng)
    write_random_model(config, tmp_path, seed=draw)
    requests = requests_for(config, 50 + draw, [41, 3, 70])
    for dtype in ("float32", "bfloat16"):
        for kind, (steps, index) in {"whole": replay_util.trace_whole(requests), "tail": replay_util.trace_tail_decode(requests, tail=12),
                                     "portions": replay_util.trace_portions(requests, sizes=(2, 31, 3, 33, 2, 16))}.items():
            runner = make_runner(tmp_path, dtype, replay_util.peak_tokens(steps), page_size=rng.choice([4, 16]))
            rows = replay_util.gather(run_steps(runner, steps), index)
            compare(rows, tmp_path, requests, dtype, f"draw {draw} {kind}")
