"""The Ditilix decoder on the device against the plain implementation (tests/plain/ditilix_plain.py):
each mechanism alone (the grouped norm that adds two branches times a factor, sinusoidal
positions, the polynomial-of-norms activation, routing by logistic scores, experts weighted at
their input, attention with a score cap and a query temperature, a layer that reads another
layer's keys and values), single keys made to decide the output against closed forms, then whole
models through the replay program (whole prompts, token-by-token decoding, prompts cut into
portions, batches of unequal requests, slots and pages used again), and greedy generation
through the library's entry point."""

import math

import numpy as np
import pytest
import torch

import ditilix_tiny as tiny
import harness
from plain import ditilix_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = ["float32", "bfloat16"]
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("ditilix_models")
    return {name: tiny.write_model(str(root / name), name) for name in tiny.CONFIGS}


# ----------------------------------------------------------------------------- comparison

_oracle = {}
_margins = {}


def oracle(folder, tokens, precision):
    key = (folder, tuple(tokens), precision)
    if key not in _oracle:
        _oracle[key] = plain.model_logits(folder, list(tokens), precision).numpy()
    return _oracle[key]


def position_error(got, want):
    """Per position: root mean square over the vocabulary of the difference, its mean taken off."""
    d = got.astype(np.float64) - want.astype(np.float64)
    d = d - d.mean(axis=1, keepdims=True)
    return np.sqrt((d * d).mean(axis=1))


def check_logits(got, folder, tokens, dtype, what):
    """float32: within a few float32 roundings of the plain float32 result.  bfloat16, against
    exact arithmetic and measured by the plain implementation's own bfloat16 emulation: the worst
    place no worse than twice the emulation's worst place, and the mean over the places no more
    than one and a half times the emulation's mean.  Places where a router's choice hangs on less
    than bfloat16's rounding of its input (in exact arithmetic) are left out; they are few."""
    assert got.shape[0] == len(tokens), f"{what}: {got.shape[0]} rows for {len(tokens)} places"
    exact = oracle(folder, tokens, torch.float64)
    spread = max(1.0, float(np.abs(exact).max()))
    if dtype == "float32":
        err = position_error(got, oracle(folder, tokens, torch.float32))
        assert err.max() <= 2e-5 * spread, f"{what}: float32 logits differ by {err.max():.3e} at place {int(err.argmax())}"
    else:
        if (folder, tuple(tokens)) not in _margins:
            _margins[(folder, tuple(tokens))] = plain.routing_margin(*plain.read_model(folder), list(tokens)).numpy()
        sure = _margins[(folder, tuple(tokens))] > 0.03
        assert sure.sum() >= 0.6 * len(tokens) - 2, f"{what}: only {int(sure.sum())} of {len(tokens)} places have a sure routing"
        noise = position_error(oracle(folder, tokens, torch.bfloat16), exact)[sure]
        err = position_error(got, exact)[sure]
        if not len(err):
            return
        worst = int(err.argmax())
        assert err.max() <= 2.0 * noise.max() + 2e-3 * spread, (
            f"{what}: bfloat16 logits are {err[worst]:.3e} from exact at place {worst}, the emulation's worst {noise.max():.3e}")
        assert err.mean() <= 1.5 * noise.mean() + 1e-3 * spread, (
            f"{what}: bfloat16 logits are {err.mean():.3e} from exact on average, the emulation {noise.mean():.3e}")


def run_trace(folder, dtype, records, tmp_path, requests, what, max_tokens=None):
    out = harness.replay(folder, dtype, records, str(tmp_path / what.replace(" ", "_")), max_tokens)
    for name, toks in requests.items():
        check_logits(out[name], folder, toks, dtype, f"{what} {name}")
    return out


def trace_portions(requests, sizes):
    """Each request alone, its tokens brought in portions of the given sizes (the last size
    repeats), logits at every place."""
    records, step = [], 0
    for name, toks in requests.items():
        at, k = 0, 0
        while at < len(toks):
            n = min(sizes[min(k, len(sizes) - 1)], len(toks) - at)
            records.append({"step": step, "entries": [{"id": name, "tokens": toks[at:at + n], "want": list(range(n))}],
                            "end": [name] if at + n == len(toks) else []})
            at, k, step = at + n, k + 1, step + 1
    return records


def rand(shape, seed, scale=1.0):
    return torch.randn(shape, generator=torch.Generator().manual_seed(seed)) * scale


def close(got, want, dtype, what):
    got, want = got.float().cpu(), want.float().cpu()
    if dtype == "float32":
        err = (got - want).abs().max().item()
        assert err <= 2e-5 * max(1.0, want.abs().max().item()), f"{what}: float32 differs by {err:.3e}"
    else:
        bad = (got - want).abs() > 2e-2 + want.abs() / 32
        assert not bad.any(), f"{what}: {int(bad.sum())} of {bad.numel()} bfloat16 values out of tolerance"


# ----------------------------------------------------------------------------- mechanisms alone


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width, groups", [(48, 1), (48, 4), (100, 5), (30, 30), (4096, 8), (5000, 2), (12288, 1), (12288, 8), (12200, 4)])
def test_grouped_norm_over_a_stream_that_takes_two_branches_and_a_factor(dtype, width, groups):
    from thing_htn_2026_b200 import ops
    t = TORCH[dtype]
    h0 = rand((6, width), 1, 2.0)
    h0[:, : width // groups] *= 30.0                       # one part far larger than the rest: shared statistics would show
    a, b = rand((6, width), 2, 3.0).to(t), rand((6, width), 3, 3.0).to(t)
    w = 1 + rand((width,), 4, 0.2)
    gain = ops.Gain(w.to(DEV), 0.0, 1e-5, groups=groups)
    # the norm alone
    _, y = ops.residual_norm(h0.clone().to(DEV), None, None, gain, t)
    close(y, plain.group_norm_rms(h0, w, groups, 1e-5), dtype, "the norm of the stream")
    # both branches times the factor, then the norm of the sum
    h = h0.clone().to(DEV)
    _, y = ops.residual_norm(h, a.to(DEV), None, gain, t, d2=b.to(DEV), mult=0.3)
    want_h = h0 + 0.3 * (a.float() + b.float())
    assert (h.cpu() - want_h).abs().max() <= 2e-6 * want_h.abs().max(), "the float32 sum"
    close(y, plain.group_norm_rms(want_h, w, groups, 1e-5), dtype, "norm of the sum")
    # one branch, a factor, no norm after it
    h = h0.clone().to(DEV)
    _, none = ops.residual_norm(h, a.to(DEV), None, None, t, mult=-1.5)
    assert none is None and (h.cpu() - (h0 - 1.5 * a.float())).abs().max() <= 2e-6 * h0.abs().max()


@pytest.mark.parametrize("width", [6, 48, 101, 1024])
def test_sinusoidal_positions_on_the_rows_of_the_embedding(width):
    from thing_htn_2026_b200 import ops
    table = rand((50, width), 5).to(torch.bfloat16)
    index = torch.tensor([3, 3, 49, 0, 7, 7, 12], dtype=torch.int32)
    positions = torch.tensor([0, 1, 2, 63, 64, 5000, 300000], dtype=torch.int32)
    pair = torch.arange((width + 1) // 2, dtype=torch.float64)
    frequencies = 10000.0 ** (-2.0 * pair / width)
    err = ops.new_error_word(DEV)
    got = ops.gather_rows_scaled(table.to(DEV), index.to(DEV), 1.0, err, positions.to(DEV), frequencies.to(DEV))
    want = table[index.long()].double() + plain.sinusoid(positions, width, torch.float64)
    assert got.dtype == torch.float32 and int(err.item()) == 0
    assert (got.cpu().double() - want).abs().max() <= 3e-7 * want.abs().max()
    # without positions the rows come out as they are
    bare = ops.gather_rows_scaled(table.to(DEV), index.to(DEV), 1.0, err)
    assert torch.equal(bare.cpu(), table[index.long()].float())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [3, 64, 77, 1000, 6000, 12288, 12250, 20000])
def test_polynomial_of_norms_alone(dtype, width):
    from thing_htn_2026_b200 import ops
    t = TORCH[dtype]
    z = rand((5, width), 6, 2.5).to(t)
    z[1] = 0                                                # a row of zeros: eps keeps it finite
    for k, coefficients in enumerate([[0.5, -0.25, 0.125, 0.1], [0.0, 1.0, 0.0, 0.0], [2.0, 0.0, 0.0, -1.0], [0.0, 0.0, 1.5, 0.0]]):
        c = torch.tensor(coefficients)
        got = ops.polynorm(z.to(DEV), c.to(DEV), 1e-5)
        close(got, plain.poly_norm(z.float(), c, 1e-5), dtype, f"coefficients {k}")


@pytest.mark.parametrize("experts, top", [(8, 1), (5, 5), (7, 3), (64, 6), (2, 1)])
def test_routing_by_logistic_scores(experts, top):
    """The largest scores, weighted by the scores themselves; logits so large that their scores
    round to one are still told apart; a router that also carries another column."""
    from thing_htn_2026_b200 import ops
    rows = 40
    z = rand((rows, experts + 1), 7, 3.0)
    z[0, :experts] = torch.arange(experts) * 3.0 + 20.0           # scores of 1.0 in float32 for all of them
    z[1, :experts] = -(torch.arange(experts) * 3.0 + 20.0)         # and of nearly nothing
    routing = ops.moe_route(z.to(DEV), experts, 1, 1, top, 1.0, scoring="logistic")
    chosen, weights = plain.route(z[:, :experts].double(), top)
    got = routing.chosen.cpu().long()
    assert torch.equal(got[1:].sort(dim=1).values, chosen[1:].sort(dim=1).values)
    # row 0: the scores are all 1.0 even in float64, the logits still order them
    assert torch.equal(got[0].sort().values, torch.arange(experts - top, experts))
    got_w = routing.chosen_weight.cpu().double()
    want_w = torch.sigmoid(z[:, :experts].double()).gather(1, got)
    assert (got_w - want_w).abs().max() <= 1e-6
    dense = routing.dense.cpu().double()
    assert (dense.gather(1, got) - want_w).abs().max() <= 1e-6
    assert ((dense != 0).sum(dim=1) <= top).all() and (dense.sum(dim=1) - want_w.sum(dim=1)).abs().max() <= 1e-5


def part_of(folder, layer_index, member, dtype):
    """One member part of a layer of a written model, built as the model builds it, with the
    checkpoint's tensors and the layer's own config entry."""
    from thing_htn_2026_b200.config import load_config
    from thing_htn_2026_b200.parts import Runtime, part_class
    from thing_htn_2026_b200.weights.loader import load_tensors
    config = load_config(folder)
    plan = config.plan()
    spec = plan.layers[plan.schedule[layer_index].layer].block.params[member]
    cls = part_class({"mixer": "mixer", "ffn": "ffn"}[member], spec.kind)
    tensors = load_tensors(folder, cls.tensor_specs(spec), TORCH[dtype], torch.device(DEV), ignored=("*",))
    runtime = Runtime(TORCH[dtype], torch.device(DEV), tensors)
    part = cls(spec, runtime)
    for shared in runtime.shared.values():
        shared.ensure(4096)
    return part, config


FEED_FORWARDS = [(name, i) for name in sorted(tiny.CONFIGS) for i, layer in enumerate(tiny.CONFIGS[name]["layers"])
                 if layer["mlp"] is not None]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name, layer", FEED_FORWARDS)
def test_feed_forward_alone(models, dtype, name, layer):
    """Every dense and routed feed-forward of the tiny models on rows large enough that the
    experts' limits cut on both sides, and on rows that are the same token scaled: with the
    routing weight on the expert's input, the output is not linear in it."""
    folder = models[name]
    part, config = part_of(folder, layer, "ffn", dtype)
    mlp = tiny.config_json(name)["layers"][layer]["mlp"]
    _, w = plain.read_model(folder)
    x = rand((33, config.width), 8 + layer, 2.0).to(TORCH[dtype])
    x[1] = x[0] * 0.25
    ar = plain.Arithmetic(torch.float32 if dtype == "float32" else torch.bfloat16)
    want = plain.feed_forward(x.float(), w, f"l{layer}.mlp.", mlp, config.norm_eps, ar)
    got = part.forward(x.to(DEV), None)
    if mlp["kind"] == "moe":
        raw = ar.linear(x.float(), w[f"l{layer}.mlp.e0.up"])
        limit = mlp["expert"]["limit"]
        assert (raw > limit).any() and (raw < -limit).any()
    if dtype == "float32":
        close(got, want, dtype, "feed-forward")
    else:
        # in bfloat16 a routing score near another may choose another expert: rows are compared by their bulk
        bad = ((got.float().cpu() - want).abs() > 3e-2 + want.abs() / 16).any(dim=1)
        assert bad.sum() <= 1, f"{int(bad.sum())} of {bad.numel()} rows differ"


class Stepper:
    """Feeds rows to a mixer that owns keys and values, and to a mixer that reads them (or
    None), through a cache of their own, as the step function would."""

    def __init__(self, owner, reader, dtype, n_slots=3):
        from thing_htn_2026_b200 import ops
        from thing_htn_2026_b200.cache import SequenceCache
        self.ops, self.owner, self.reader = ops, owner, reader
        assert reader is None or reader.cache_need() is None
        self.cache = SequenceCache([owner.cache_need()], max_tokens=64 * 40, dtype=TORCH[dtype], device=DEV,
                                   max_slots=n_slots)
        self.err = ops.new_error_word(DEV)

    def step(self, slots, xs, ys=None):
        """xs[i]: rows [n_i, width] that slot i brings to the owner; ys[i]: the rows it brings
        to the reader.  Returns the owner's rows per slot (and the reader's)."""
        from thing_htn_2026_b200.config.base import ScheduleEntry
        from thing_htn_2026_b200.parts import HostBatch, StepContext
        ops, cache = self.ops, self.cache
        counts = [x.shape[0] for x in xs]
        cache.prepare(slots, counts)
        held = [cache.length(s) for s in slots]
        cu = [0]
        for c in counts:
            cu.append(cu[-1] + c)
        cu_dev = torch.tensor(cu, dtype=torch.int32, device=DEV)
        slots_dev = torch.tensor(slots, dtype=torch.int32, device=DEV)
        rows = ops.step_rows(cu_dev, slots_dev, cache.seq_lens, cu[-1], max(counts))
        asked = {}
        self.owner.step_inputs(HostBatch(slots, counts, held, cache.page_size), asked)
        if self.reader is not None:
            self.reader.step_inputs(HostBatch(slots, counts, held, cache.page_size), asked)
        inputs = {k: torch.tensor(v, dtype=torch.int32, device=DEV) for k, v in asked.items()}
        ctx = StepContext(rows=rows, cache=cache, err=self.err, inputs=inputs)
        a = self.owner.forward(torch.cat(xs).to(DEV).contiguous(), ctx, ScheduleEntry(0, 0))
        b = None
        if self.reader is not None:
            b = self.reader.forward(torch.cat(ys).to(DEV).contiguous(), ctx, ScheduleEntry(1, 0, writes_cache=False))
        ops.advance(cache.seq_lens, slots_dev, cu_dev)
        cache.commit(slots, counts)
        assert int(self.err.item()) == 0
        cut = lambda t: None if t is None else [t[lo:hi] for lo, hi in zip(cu[:-1], cu[1:])]
        return cut(a), cut(b)


# (model, the layer that owns keys and values, a layer that reads them or None)
MIXER_PAIRS = [("a", 0, 3), ("a", 1, 2), ("b", 0, 1), ("b", 2, None), ("c", 0, 1), ("c", 2, 3), ("d", 0, 1), ("d", 2, None)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name, own, reads", MIXER_PAIRS)
def test_mixers_alone_whole_in_portions_and_token_by_token(models, dtype, name, own, reads):
    """A mixer with keys of its own and one that reads them, against the plain mechanism, for a
    sequence brought whole, in portions of unequal sizes down to two and one, beside another
    sequence, and in a slot that was used before."""
    folder = models[name]
    owner, config = part_of(folder, own, "mixer", dtype)
    reader = part_of(folder, reads, "mixer", dtype)[0] if reads is not None else None
    layers = tiny.config_json(name)["layers"]
    _, w = plain.read_model(folder)
    ar = plain.Arithmetic(torch.float32 if dtype == "float32" else torch.bfloat16)
    t = TORCH[dtype]
    T = 150

    def plainly(x, y):
        kv = plain.project_kv(x.float(), w, f"l{own}.mix.", layers[own]["mixer"], ar)
        a = plain.attention_mixer(x.float(), w, f"l{own}.mix.", layers[own]["mixer"], ar, kv)
        b = plain.attention_mixer(y.float(), w, f"l{reads}.mix.", layers[reads]["mixer"], ar, kv) if reads is not None else None
        return a, b

    x, y = rand((T, config.width), 100 + own).to(t), rand((T, config.width), 150 + own).to(t)
    ox, oy = rand((31, config.width), 200 + own).to(t), rand((31, config.width), 250 + own).to(t)
    want, want_other = plainly(x, y), plainly(ox, oy)

    def check(got, wanted, what):
        close(torch.cat(got[0]), wanted[0], dtype, what + ", own keys")
        if reads is not None:
            close(torch.cat(got[1]), wanted[1], dtype, what + ", another layer's keys")

    stepper = Stepper(owner, reader, dtype)
    s0, s1, s2 = stepper.cache.open(3)
    whole = stepper.step([s0], [x], [y])
    check(whole, want, "whole")
    cuts = [0, 3, 5, 63, 64, 66, 128, 130, 131, 132, T]
    got, got_other, at = ([], []), ([], []), 0
    for lo, hi in zip(cuts[:-1], cuts[1:]):
        if at < ox.shape[0]:
            n = min(hi - lo + 1, ox.shape[0] - at)
            a, b = stepper.step([s2, s1], [ox[at:at + n], x[lo:hi]], [oy[at:at + n], y[lo:hi]])
            got_other[0].append(a[0]), got[0].append(a[1])
            if reads is not None:
                got_other[1].append(b[0]), got[1].append(b[1])
            at += n
        else:
            a, b = stepper.step([s1], [x[lo:hi]], [y[lo:hi]])
            got[0].append(a[0])
            if reads is not None:
                got[1].append(b[0])
    check(got, want, "in portions")
    check(got_other, want_other, "the sequence beside it")
    if dtype == "float32":
        # what a position gets must not depend on the cut beyond rounding
        assert (torch.cat(got[0]) - whole[0][0]).abs().max() <= 2e-5 * max(1.0, whole[0][0].abs().max().item())
    stepper.cache.close([s0])
    (again,) = stepper.cache.open(1)
    assert again == s0
    check(stepper.step([again], [ox], [oy]), want_other, "a slot used again")


# ----------------------------------------------------------------------------- single keys made to show


def factor_at(p, coef, every):
    """The query temperature at positions p (float64)."""
    if not every:
        return np.ones_like(p, dtype=np.float64)
    return 1.0 + coef * np.log(np.floor((p + 1) / every) + 1.0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d, dv, n_q, n_kv, spare", [(16, 16, 2, 1, 0), (64, 64, 4, 2, 8), (48, 32, 3, 3, 0), (20, 36, 2, 1, 4),
                                                    (128, 128, 2, 1, 0), (9, 5, 2, 2, 1), (24, 40, 1, 1, 3), (12, 12, 5, 1, 0)])
def test_projected_rows_are_split_untouched(dtype, d, dv, n_q, n_kv, spare):
    """Without norm and rotation `ops.qk_prepare` only splits a projected row: the queries come
    back and the keys and values lie in the cache, bit for bit, at the positions of two sequences
    of unequal lengths that cross a page border.  Sizes that allow 16-byte pieces and sizes that do
    not (odd ones, rows with spare entries that break the alignment of the next row)."""
    from thing_htn_2026_b200 import ops
    from thing_htn_2026_b200.cache import KVSpec, SequenceCache
    t = TORCH[dtype]
    lens = [70, 3]
    width = n_q * d + n_kv * (d + dv) + spare
    g = torch.Generator().manual_seed(d * 100 + dv)
    proj = torch.randn(sum(lens), width, generator=g).to(t)
    cache = SequenceCache([KVSpec(n_kv, d, value_dim=dv)], max_tokens=64 * 4, dtype=t, device=DEV, max_slots=2)
    slots = cache.open(2)
    cache.prepare(slots, lens)
    cu = torch.tensor([0, lens[0], sum(lens)], dtype=torch.int32, device=DEV)
    rows = ops.step_rows(cu, torch.tensor(slots, dtype=torch.int32, device=DEV), cache.seq_lens, sum(lens), max(lens))
    err = ops.new_error_word(DEV)
    kv = cache.kv_view(0)
    q = ops.qk_prepare(proj.to(DEV), None, None, None, 1.0, None, rows, kv, n_q, False, True, err)
    assert int(err.item()) == 0
    assert torch.equal(q.cpu(), proj[:, :n_q * d]), "queries"
    storage = kv.storage.cpu().reshape(kv.storage.shape[0], -1)
    page = kv.page_size
    row = 0
    for slot, n in zip(slots, lens):
        pages = cache.book.pages_of(0, slot)
        for pos in range(n):
            flat = storage[pages[pos // page]]
            keys = flat[:n_kv * page * d].reshape(n_kv, page, d)[:, pos % page]
            values = flat[n_kv * page * d:].reshape(n_kv, page, dv)[:, pos % page]
            assert torch.equal(keys.reshape(-1), proj[row, n_q * d:(n_q + n_kv) * d]), f"keys of position {pos}"
            assert torch.equal(values.reshape(-1), proj[row, (n_q + n_kv) * d:(n_q + n_kv) * d + n_kv * dv]), f"values of position {pos}"
            row += 1


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d, dv, n_q, n_kv", [(16, 16, 2, 1), (64, 64, 4, 2), (48, 32, 3, 3), (20, 36, 2, 1), (128, 128, 2, 1)])
@pytest.mark.parametrize("cap, coef, every", [(0.0, 0.0, 0), (0.0, -0.02, 1), (2.5, 0.0, 0), (4.0, 0.5, 16), (3.0, 1.0, 70)])
def test_one_loud_key_among_hundreds_against_the_closed_form(dtype, d, dv, n_q, n_kv, cap, coef, every):
    """Keys and values are written as they are.  All keys of a sequence are small but one, every
    query is all ones and every value row is its own position, so the raw score of a key is 30
    (the loud one) or 30/128 times the query's temperature, and what a query returns follows in
    closed form: without a cap the loud key alone, wherever it lies (the first token, a page's
    last and first place, hundreds of places back), or the mean position before it appears; with
    a cap a mixture whose weights depend on the cap, on the temperature, and on the cap coming
    after the temperature.  Several sequences, each with its loud key elsewhere, run as one
    batch: as a whole prompt, and with the second half decoded one token a step."""
    from thing_htn_2026_b200 import ops
    from thing_htn_2026_b200.cache import KVSpec, SequenceCache
    t = TORCH[dtype]
    L, small = 300, 1.0 / 128
    louds = [0, 1, 63, 64, 127, 128, 149, 150, 200, 299]
    S = len(louds)
    cache = SequenceCache([KVSpec(n_kv, d, value_dim=dv)], max_tokens=64 * 5 * S, dtype=t, device=DEV, max_slots=S)
    kv = cache.kv_view(0)
    err = ops.new_error_word(DEV)
    k = torch.full((S, L, n_kv, d), small)
    for s, loud in enumerate(louds):
        k[s, loud] = 1.0
    v = (torch.arange(L, dtype=torch.float32) / 64.0)[None, :, None, None].expand(S, L, n_kv, dv)
    proj = torch.cat([torch.ones(S, L, n_q * d), k.reshape(S, L, -1), v.reshape(S, L, -1)], dim=2).to(t)
    shape = ops.ScoreShape(cap, coef, every)
    tile = ops.prompt_attention_tile(t, d, cache.page_size, n_q, n_kv, dv, None)
    i = np.arange(L)

    def expected(loud):
        raw = np.where(i[None, :] == loud, 30.0, 30.0 * small) * factor_at(i, coef, every)[:, None]   # [query, key]
        if cap:
            raw = cap * np.tanh(raw / cap)
        raw = np.where(i[None, :] <= i[:, None], raw, -np.inf)
        weights = np.exp(raw - raw.max(axis=1, keepdims=True))
        return (weights * i[None, :]).sum(axis=1) / weights.sum(axis=1) / 64.0

    for prompt_len in (L, 150):
        slots = cache.open(S)
        outs, at = [[] for _ in range(S)], 0
        for n in [prompt_len] + [1] * (L - prompt_len):
            cache.prepare(slots, [n] * S)
            cu = torch.tensor([n * j for j in range(S + 1)], dtype=torch.int32, device=DEV)
            sl = torch.tensor(slots, dtype=torch.int32, device=DEV)
            rows = ops.step_rows(cu, sl, cache.seq_lens, n * S, n, max_context=L)
            x = proj[:, at:at + n].reshape(S * n, -1).to(DEV).contiguous()
            q = ops.qk_prepare(x, None, None, None, 1.0, None, rows, kv, n_q, False, True, err)
            tiles = None
            if n > 1 and tile:
                r0, rr = ops.row_tiles_of([n] * S, [at] * S, tile)
                tiles = ops.RowTiles(torch.tensor(r0, dtype=torch.int32, device=DEV),
                                     torch.tensor(rr, dtype=torch.int32, device=DEV), len(r0), tile)
            a = ops.attention(q, rows, kv, n_q, 30.0 / d, None, err, tiles, shape=shape).float().cpu().reshape(S, n, n_q, dv)
            for s in range(S):
                outs[s].append(a[s])
            ops.advance(cache.seq_lens, sl, cu)
            cache.commit(slots, [n] * S)
            at += n
        assert int(err.item()) == 0
        for s, loud in enumerate(louds):
            out = torch.cat(outs[s]).numpy()                         # [L, n_q, dv]
            want = expected(loud)
            if not cap:
                assert np.abs(want[loud:] - loud / 64.0).max() < 1e-6   # the loud key alone, once it is there
            tolerance = (1e-4 if dtype == "float32" else 6e-3) * np.maximum(1.0, want) + (1e-4 if dtype == "float32" else 4e-3)
            wrong = np.abs(out - want[:, None, None]).max(axis=(1, 2)) > tolerance
            assert not wrong.any(), (
                f"loud key {loud}, prompt of {prompt_len}: queries {i[wrong][:8].tolist()} got "
                f"{(out[wrong][:8, 0, 0] * 64).round(3).tolist()}, expected {(want[wrong][:8] * 64).round(3).tolist()}")
        cache.close(slots)


def test_the_closed_form_tells_the_options_apart():
    """What the test above compares with moves by far more than its tolerance when the cap comes
    before the temperature or is left out, and by ten times its float32 tolerance when the
    temperature's period starts one position late: a kernel that did any of these would not pass."""
    i = np.arange(300)

    def mixture(raw, cap):
        raw = cap * np.tanh(raw / cap) if cap else raw
        raw = np.where(i[None, :] <= i[:, None], raw, -np.inf)
        w = np.exp(raw - raw.max(axis=1, keepdims=True))
        return (w * i[None, :]).sum(axis=1) / w.sum(axis=1) / 64.0

    base = np.where(i[None, :] == 64, 30.0, 30.0 / 128)
    right = mixture(base * factor_at(i, 0.5, 16)[:, None], 4.0)
    late = mixture(base * factor_at(i - 1, 0.5, 16)[:, None], 4.0)
    swapped = mixture(4.0 * np.tanh(base / 4.0) * factor_at(i, 0.5, 16)[:, None], 0.0)
    bare = mixture(base * factor_at(i, 0.5, 16)[:, None], 0.0)
    assert np.abs(late - right).max() > 1.5e-3
    assert np.abs(swapped - right).max() > 0.5 and np.abs(bare - right).max() > 0.5


# ----------------------------------------------------------------------------- whole models


def requests_of(name, lengths, seed):
    return {f"r{n}": tiny.tokens(name, n, seed + n) for n in lengths}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_whole_prompts_and_their_first_tokens(models, tmp_path, dtype, name):
    requests = requests_of(name, [1, 2, 3, 64, 65, 211], 10)
    run_trace(models[name], dtype, harness.trace_whole(requests), tmp_path, requests, "whole")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_decoding_token_by_token_long(models, tmp_path, dtype, name):
    """A prompt of 40 and 190 tokens decoded one by one: the temperature passes several of its
    steps over decoded tokens, and layers that read another layer's keys find them page after page."""
    requests = requests_of(name, [230], 20)
    run_trace(models[name], dtype, harness.trace_tail(requests, tail=190), tmp_path, requests, "decoded")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_prompts_in_portions(models, tmp_path, dtype, name):
    requests = requests_of(name, [150], 30)
    for sizes in ([2], [63, 2, 1, 64, 3], [5, 100, 2, 2, 7]):
        run_trace(models[name], dtype, trace_portions(requests, sizes), tmp_path, requests, f"portions {sizes[0]}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_batches_of_unequal_requests(models, tmp_path, dtype, name):
    """Two batches, one after the other, in a cache that holds one of them: the second batch
    takes the slots and pages that the first gave back.  Every request also alone."""
    first = requests_of(name, [1, 70, 135, 23], 40)
    second = {k + "x": v for k, v in requests_of(name, [90, 2, 140], 50).items()}
    prompt_lens = {"r1": 1, "r70": 50, "r135": 100, "r23": 23, "r90x": 64, "r2x": 1, "r140x": 128}
    records = harness.trace_batches([first, second], prompt_lens)
    together = run_trace(models[name], dtype, records, tmp_path, {**first, **second}, "batches",
                         max_tokens=harness.max_tokens_of(records))
    alone = harness.replay(models[name], dtype, harness.trace_whole({**first, **second}), str(tmp_path / "alone"))
    if dtype == "float32":
        for key in together:
            err = position_error(together[key], alone[key])
            assert err.max() <= 3e-5 * max(1.0, np.abs(alone[key]).max()), f"{key}: a batch and the request alone differ by {err.max():.3e}"


@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_the_stream_after_every_layer(models, name):
    """The float32 residual stream after each layer of a short prompt (the stream a layer hands
    on, plus the branches it has not added yet times their factor), through the model's own
    layers and cache, against the plain implementation's."""
    from thing_htn_2026_b200 import ops
    from thing_htn_2026_b200.cache import SequenceCache
    from thing_htn_2026_b200.engine.loading import load_model
    from thing_htn_2026_b200.parts import HostBatch, StepContext
    toks = tiny.tokens(name, 37, 5)
    config, tensors = plain.read_model(models[name])
    want = []
    plain.forward(config, tensors, toks, torch.float32, layers_out=want)
    with torch.inference_mode():
        model = load_model(models[name], "float32", DEV)
        cache = SequenceCache(model.cache_needs(), max_tokens=128, dtype=torch.float32, device=DEV)
        (slot,) = cache.open(1)
        n = len(toks)
        cache.prepare([slot], [n])
        model.ensure_positions(n)
        cu = torch.tensor([0, n], dtype=torch.int32, device=DEV)
        slots = torch.tensor([slot], dtype=torch.int32, device=DEV)
        asked = model.step_inputs(HostBatch([slot], [n], [0], cache.page_size))
        inputs = {k: torch.tensor(v, dtype=torch.int32, device=DEV) for k, v in asked.items()}
        err = ops.new_error_word(DEV)
        ctx = StepContext(rows=ops.step_rows(cu, slots, cache.seq_lens, n, n, max_context=n), cache=cache, err=err,
                          inputs=inputs)
        h, d = model.embedding.forward(torch.tensor(toks, dtype=torch.int32, device=DEV), err, ctx.rows), None
        assert h.dtype == torch.float32
        for k, entry in enumerate(model.plan.schedule):
            h, d = model.layers[entry.layer].forward(h, d, ctx, entry)
            pending = d.tensor.float() + (d.second.float() if d.second is not None else 0.0)
            got = (h + d.factor * pending).cpu()
            worst = (got - want[k]).abs().max().item()
            assert worst <= 2e-5 * max(1.0, want[k].abs().max().item()), f"after layer {k}: the stream differs by {worst:.3e}"
        assert int(err.item()) == 0


def test_what_the_plain_implementation_would_show(models):
    """The plain implementation moves far when a layer that reads another layer's keys is given
    keys of its own input instead, when the routing weight goes to the expert's output, and when
    positions start at 1: the comparisons above would notice any of these."""
    name = "a"
    config, tensors = plain.read_model(models[name])
    toks = tiny.tokens(name, 60, 77)
    right = plain.forward(config, tensors, toks, torch.float64).numpy()
    shifted = plain.forward(config, tensors, [toks[0]] + toks, torch.float64).numpy()[1:]
    assert position_error(right[1:], shifted[1:]).min() > 1e-3
    n = torch.randn(20, config["width"], generator=torch.Generator().manual_seed(1), dtype=torch.float64)
    ar = plain.Arithmetic(torch.float64)
    mlp = config["layers"][1]["mlp"]
    t = {k: v.double() for k, v in tensors.items()}
    inside = plain.moe(n, t, "l1.mlp.", mlp, ar)
    z = ar.linear(n, t["l1.mlp.router"], keep=True)
    chosen, weights = plain.route(z, mlp["router"]["top"])
    outside = torch.zeros_like(n)
    for r in range(n.shape[0]):
        for e, w in zip(chosen[r].tolist(), weights[r].tolist()):
            outside[r] += w * plain.clamped_expert(n[r:r + 1], t, f"l1.mlp.e{e}.", mlp["expert"]["limit"], ar)[0]
    gate = torch.sigmoid(ar.linear(n, t["l1.mlp.shared.sg"], keep=True))
    outside += gate * plain.clamped_expert(n, t, "l1.mlp.shared.", mlp["shared"]["limit"], ar)
    assert (inside - outside).abs().max() > 1e-2


def greedy_by_plain(folder, prompt, n_new):
    config, tensors = plain.read_model(folder)
    seq, margins = list(prompt), []
    for _ in range(n_new):
        logits = plain.forward(config, tensors, seq, torch.float64)[-1]
        top = logits.topk(2).values
        margins.append(float(top[0] - top[1]))
        seq.append(int(logits.argmax()))
    return seq[len(prompt):], margins


@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("name", ["a", "c"])
def test_greedy_generation_through_the_engine(models, name, graphs):
    """Engine.generate: the library's own entry point, scheduler, captured decode step and token
    choice, on prompts of unequal lengths, against greedy continuation by the plain
    implementation (up to the first step whose two best logits are closer than rounding)."""
    from thing_htn_2026_b200 import Engine
    prompts = [tiny.tokens(name, n, 50 + n) for n in (5, 70, 23)]
    new = 20
    engine = Engine(models[name], dtype="float32", graphs=graphs)
    got = [[] for _ in prompts]
    for step in engine.generate(prompts, new):
        for i, token in enumerate(step):
            got[i].append(token)
    compared = 0
    for i, prompt in enumerate(prompts):
        want, margins = greedy_by_plain(models[name], prompt, new)
        sure = next((k for k, m in enumerate(margins) if m < 3e-4), new)
        assert got[i][:sure] == want[:sure], f"prompt {i}: {got[i]} against {want} (sure of the first {sure})"
        compared += sure
    assert compared >= 24
    again = [[] for _ in prompts]
    for step in engine.generate(prompts, 6):
        for i, token in enumerate(step):
            again[i].append(token)
    assert [a[:6] for a in again] == [g[:6] for g in got]


def test_generation_in_bfloat16_runs_and_stays_in_the_vocabulary(models):
    from thing_htn_2026_b200 import Engine
    engine = Engine(models["b"], dtype="bfloat16")
    prompts = [tiny.tokens("b", n, 60 + n) for n in (3, 40)]
    steps = list(engine.generate(prompts, 12, temperature=[0.0, 0.8], seed=3))
    assert len(steps) == 12 and all(0 <= t < 300 for step in steps for t in step)
