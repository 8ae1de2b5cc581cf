"""The Dubazen decoder on the device against the plain implementation (tests/plain/dubazen_plain.py):
each mechanism alone (the streams' write, read and norm in one kernel; routing by a renormalised
softmax and experts weighted at their output; attention with biases, turned values, a sink and a
gate; linear attention with constant and with gated decays; the pair of mixers that share their
products; the selective scan behind its convolution), single keys made to decide the output against
closed forms, then whole models through the replay program (whole prompts, token-by-token decoding,
prompts cut into portions, batches of unequal requests, slots and pages used again), and greedy
generation through the library's entry point."""

import math

import numpy as np
import pytest
import torch

import dubazen_tiny as tiny
import harness
from plain import dubazen_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = ["float32", "bfloat16"]
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("dubazen_models")
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
    """float32: within a few float32 roundings of the plain float32 result.  bfloat16, against exact
    arithmetic and measured by the plain implementation's own bfloat16 emulation: the worst place no
    worse than twice the emulation's worst place, the mean no more than one and a half times its
    mean.  Places where a router's choice hangs on less than 0.08 in its logits (in exact
    arithmetic) are left out of the bfloat16 comparison, and so are the sixteen places behind each:
    a recurrent layer carries another expert's output on for a while."""
    assert got.shape[0] == len(tokens), f"{what}: {got.shape[0]} rows for {len(tokens)} places"
    exact = oracle(folder, tokens, torch.float64)
    spread = max(1.0, float(np.abs(exact).max()))
    if dtype == "float32":
        err = position_error(got, oracle(folder, tokens, torch.float32))
        assert err.max() <= 3e-5 * spread, f"{what}: float32 logits differ by {err.max():.3e} at place {int(err.argmax())}"
        return
    if (folder, tuple(tokens)) not in _margins:
        _margins[(folder, tuple(tokens))] = plain.routing_margin(folder, list(tokens)).numpy()
    sure = np.ones(len(tokens), dtype=bool)
    for place in np.nonzero(_margins[(folder, tuple(tokens))] <= 0.08)[0]:
        sure[place:place + 17] = False
    if not sure.any():
        return
    noise = position_error(oracle(folder, tokens, torch.bfloat16), exact)[sure]
    err = position_error(got, exact)[sure]
    worst = int(err.argmax())
    assert err.max() <= 2.0 * noise.max() + 3e-3 * spread, (
        f"{what}: bfloat16 logits are {err[worst]:.3e} from exact at place {worst}, the emulation's worst {noise.max():.3e}")
    assert err.mean() <= 1.5 * noise.mean() + 1.5e-3 * spread, (
        f"{what}: bfloat16 logits are {err.mean():.3e} from exact on average, the emulation {noise.mean():.3e}")


def run_trace(folder, dtype, records, tmp_path, requests, what, max_tokens=None):
    out = harness.replay(folder, dtype, records, str(tmp_path / what.replace(" ", "_")), max_tokens)
    for name, toks in requests.items():
        check_logits(out[name], folder, toks, dtype, f"{what} {name}")
    return out


def trace_portions(requests, sizes):
    """Each request alone, its tokens brought in portions of the given sizes (the last size repeats)."""
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


def close(got, want, dtype, what, loose=1.0):
    got, want = got.float().cpu(), want.float().cpu()
    if dtype == "float32":
        err = (got - want).abs().max().item()
        assert err <= 3e-5 * loose * max(1.0, want.abs().max().item()), f"{what}: float32 differs by {err:.3e}"
    else:
        bad = (got - want).abs() > loose * (3e-2 * max(1.0, want.abs().max().item() / 4) + want.abs() / 16)
        assert bad.sum() <= bad.numel() // 200, f"{what}: {int(bad.sum())} of {bad.numel()} bfloat16 values out of tolerance"


# ----------------------------------------------------------------------------- the streams


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("streams, width, vector", [(1, 40, False), (2, 100, False), (3, 48, True), (4, 256, False),
                                                    (5, 30, False), (16, 72, False), (4, 4096, False), (3, 12288, True)])
def test_write_read_and_norm_over_the_streams(dtype, streams, width, vector):
    """hyper_norm in its three places: at the start (every copy is the embedding's row), between two
    sublayers (the write of one, the read of the next), and at the end (the write, then the sum of
    the copies); the mix matrix is far from symmetric, so that [from, to] read the other way shows."""
    from thing_htn_2026_b200 import ops
    rows, t = 7, TORCH[dtype]
    x0 = rand((rows, width), 1, 3.0)
    y = rand((rows, width), 2).to(t)
    read, write, mix = rand((streams,), 3), rand((streams,), 4), rand((streams, streams), 5)
    gain = rand((width,), 6).abs() + 0.5 if vector else torch.tensor([1.7])
    eps = 1e-5
    norm = lambda u: u / torch.sqrt((u * u).mean(-1, keepdim=True) + eps) * gain
    dev = lambda v: v.to(DEV).contiguous()
    X, n = ops.hyper_norm(None, streams, t, start=dev(x0), read=dev(read), gain=dev(gain), eps=eps)
    assert torch.equal(X.cpu().view(rows, streams, width), x0[:, None, :].expand(rows, streams, width))
    close(n, norm(x0 * read.sum()), dtype, "the start")
    Xs = rand((rows, streams, width), 7, 2.0)
    want_X = torch.einsum("ji,tjw->tiw", mix, Xs) + write[None, :, None] * y.float()[:, None, :]
    numbers = ops.StreamNumbers(dev(read), dev(mix), dev(write))
    X, n = ops.hyper_norm(dev(Xs.reshape(rows, -1)), streams, t, y=dev(y), written=numbers, read=dev(read), gain=dev(gain), eps=eps)
    assert (X.cpu().view(rows, streams, width) - want_X).abs().max() <= 1e-5 * want_X.abs().max()
    close(n, norm(torch.einsum("j,tjw->tw", read, want_X)), dtype, "between two sublayers")
    X, n = ops.hyper_norm(dev(Xs.reshape(rows, -1)), streams, t, y=dev(y), written=numbers, read=dev(torch.ones(streams)),
                          gain=dev(gain), eps=eps)
    close(n, norm(want_X.sum(1)), dtype, "the end")
    if streams > 1:
        wrong = norm(torch.einsum("j,tjw->tw", read, torch.einsum("ij,tjw->tiw", mix, Xs) + write[None, :, None] * y.float()[:, None, :]))
        assert (wrong - norm(torch.einsum("j,tjw->tw", read, want_X))).abs().max() > 0.05
    X, n = ops.hyper_norm(dev(Xs.reshape(rows, -1)), streams, t, y=dev(y), written=numbers)
    assert n is None and (X.cpu().view(rows, streams, width) - want_X).abs().max() <= 1e-5 * want_X.abs().max()


# ----------------------------------------------------------------------------- routing and experts


@pytest.mark.parametrize("experts, top", [(8, 1), (5, 5), (7, 3), (64, 6), (2, 1), (16, 3)])
def test_routing_by_a_renormalised_softmax(experts, top):
    from thing_htn_2026_b200 import ops
    z = rand((50, experts), experts + top, 3.0)
    z[0] = 0.0                     # all equal: the lowest indices win
    z[1, :] = -80.0
    z[1, experts - 1] = 80.0       # one score that is 1 in float32 and others that are 0
    routing = ops.moe_route(z.to(DEV), experts, 1, 1, top, 1.0, scoring="softmax", renormalise=1e-20)
    s = torch.softmax(z.double(), -1)
    best = torch.topk(s, top, dim=-1)
    want = torch.zeros(50, experts, dtype=torch.float64)
    want.scatter_(1, best.indices, best.values / (best.values.sum(-1, keepdim=True) + 1e-20))
    got = routing.dense.cpu().double()
    assert sorted(routing.chosen[0].tolist()) == list(range(top))
    rows = [r for r in range(50) if r != 0]
    assert (got[rows] - want[rows]).abs().max() < 1e-6
    assert torch.allclose(got.sum(-1), torch.ones(50, dtype=torch.float64), atol=1e-6)
    plain_weights = ops.moe_route(z.to(DEV), experts, 1, 1, top, 1.0, scoring="softmax").dense.cpu().double()
    if top < experts:
        assert (plain_weights.sum(-1) < 0.999).any()       # without the division the weights do not sum to one


def part_of(folder, layer_index, member, dtype):
    """One member part of a layer of a written model, built as the model builds it."""
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
    """Every feed-forward of the tiny models on rows large enough that the experts' limits cut on
    both sides; the weight on the output makes the routed part linear in it, which the plain
    implementation computes expert by expert."""
    import warnings
    folder = models[name]
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        part, config = part_of(folder, layer, "ffn", dtype)
    mlp = tiny.config_json(name)["layers"][layer]["mlp"]
    _, w = plain.read_model(folder)
    x = rand((33, config.width), 8 + layer, 2.0).to(TORCH[dtype])
    ar = plain.Arithmetic(torch.float32 if dtype == "float32" else torch.bfloat16)
    want = plain.mixture(ar, x.float(), w, f"l{layer}.mlp.", mlp)
    got = part.forward(x.to(DEV), None)
    raw = ar.linear(x.float(), w[f"l{layer}.mlp.e0.up"])
    assert (raw > mlp["expert"]["limit"]).any() and (raw < -mlp["expert"]["limit"]).any()
    if dtype == "float32":
        close(got, want, dtype, "feed-forward")
    else:
        bad = ((got.float().cpu() - want).abs() > 3e-2 + want.abs() / 16).any(dim=1)
        assert bad.sum() <= 2, f"{int(bad.sum())} of {bad.numel()} rows differ"


# ----------------------------------------------------------------------------- mixers alone


class Stepper:
    """Feeds rows to a mixer through a cache of its own, as the step function would."""

    def __init__(self, mixer, dtype, n_slots=3):
        from thing_htn_2026_b200 import ops
        from thing_htn_2026_b200.cache import SequenceCache
        self.ops, self.mixer = ops, mixer
        self.cache = SequenceCache([mixer.cache_need()], max_tokens=64 * 40, dtype=TORCH[dtype], device=DEV, max_slots=n_slots)
        self.err = ops.new_error_word(DEV)

    def step(self, slots, xs):
        from thing_htn_2026_b200.config.base import ScheduleEntry
        from thing_htn_2026_b200.parts import StepContext
        ops, cache = self.ops, self.cache
        counts = [x.shape[0] for x in xs]
        cache.prepare(slots, counts)
        cu = [0]
        for c in counts:
            cu.append(cu[-1] + c)
        cu_dev = torch.tensor(cu, dtype=torch.int32, device=DEV)
        slots_dev = torch.tensor(slots, dtype=torch.int32, device=DEV)
        rows = ops.step_rows(cu_dev, slots_dev, cache.seq_lens, cu[-1], max(counts))
        ctx = StepContext(rows=rows, cache=cache, err=self.err, inputs={})
        a = self.mixer.forward(torch.cat(xs).to(DEV).contiguous(), ctx, ScheduleEntry(0, 0))
        ops.advance(cache.seq_lens, slots_dev, cu_dev)
        cache.commit(slots, counts)
        assert int(self.err.item()) == 0
        return [a[lo:hi] for lo, hi in zip(cu[:-1], cu[1:])]


def plain_mixer(folder, name, layer, x, ar):
    config, w = plain.read_model(folder)
    entry = config["layers"][layer]
    prefix, eps = f"l{layer}.mix.", config["norm"]["eps"]
    if entry["type"] == "parallel":
        return plain.parallel_mixer(ar, x, w, prefix, entry["mixer"], eps, torch.arange(x.shape[0]))
    if entry["type"] == "gla":
        return plain.gated_linear_attention(ar, x, w, prefix, entry["mixer"], eps)
    return plain.selective_scan(ar, x, w, prefix, entry["mixer"])


MIXERS = [(name, i) for name in sorted(tiny.CONFIGS) for i in range(len(tiny.CONFIGS[name]["layers"]))]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name, layer", MIXERS)
def test_mixers_alone_whole_in_portions_and_token_by_token(models, dtype, name, layer):
    """Every mixer of the tiny models against the plain mechanism, for a sequence brought whole, in
    portions of unequal sizes down to two and one (shorter than the convolution's taps, across page
    borders), beside another sequence, token by token at its end, and in a slot that was used before
    (its state and ring must start from zero again)."""
    import warnings
    folder = models[name]
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        mixer, config = part_of(folder, layer, "mixer", dtype)
    ar = plain.Arithmetic(torch.float32 if dtype == "float32" else torch.bfloat16)
    t = TORCH[dtype]
    T = 150
    x, ox = rand((T, config.width), 100 + layer).to(t), rand((31, config.width), 200 + layer).to(t)
    want, want_other = plain_mixer(folder, name, layer, x.float(), ar), plain_mixer(folder, name, layer, ox.float(), ar)
    stepper = Stepper(mixer, dtype)
    s0, s1, s2 = stepper.cache.open(3)
    whole = stepper.step([s0], [x])
    close(whole[0], want, dtype, "whole")
    cuts = [0, 1, 3, 5, 63, 64, 66, 128, 130] + list(range(131, T + 1))
    got, got_other, at = [], [], 0
    for lo, hi in zip(cuts[:-1], cuts[1:]):
        if at < ox.shape[0]:
            n = min(hi - lo + 1, ox.shape[0] - at)
            a = stepper.step([s2, s1], [ox[at:at + n], x[lo:hi]])
            got_other.append(a[0]), got.append(a[1])
            at += n
        else:
            got.append(stepper.step([s1], [x[lo:hi]])[0])
    close(torch.cat(got), want, dtype, "in portions and token by token")
    close(torch.cat(got_other), want_other, dtype, "the sequence beside it")
    if dtype == "float32":
        # what a position gets must not depend on the cut beyond rounding
        assert (torch.cat(got) - whole[0]).abs().max() <= 2e-5 * max(1.0, whole[0].abs().max().item())
    stepper.cache.close([s0])
    (again,) = stepper.cache.open(1)
    assert again == s0
    close(stepper.step([again], [ox])[0], want_other, dtype, "a slot used again")


# ----------------------------------------------------------------------------- single keys made to show


class KeysAndValues:
    """A cache entry of keys and values filled through the library's own preparation kernel."""

    def __init__(self, n_kv, d, dv, dtype):
        from thing_htn_2026_b200 import ops
        from thing_htn_2026_b200.cache import SequenceCache
        from thing_htn_2026_b200.cache.sequence_cache import KVSpec
        self.ops = ops
        self.cache = SequenceCache([KVSpec(n_kv, d, None, 0, None, dv)], max_tokens=64 * 12, dtype=TORCH[dtype], device=DEV, max_slots=2)
        self.err = ops.new_error_word(DEV)
        (self.slot,) = self.cache.open(1)

    def rows(self, count):
        ops, cache = self.ops, self.cache
        cache.prepare([self.slot], [count])
        self.cu = torch.tensor([0, count], dtype=torch.int32, device=DEV)
        self.slots = torch.tensor([self.slot], dtype=torch.int32, device=DEV)
        return ops.step_rows(self.cu, self.slots, cache.seq_lens, count, count)

    def done(self, count):
        self.ops.advance(self.cache.seq_lens, self.slots, self.cu)
        self.cache.commit([self.slot], [count])
        assert int(self.err.item()) == 0


def rope_tables(dim, base, layout="half", n=1024):
    from thing_htn_2026_b200 import ops
    angle = torch.arange(n, dtype=torch.float64)[:, None] * base ** (-torch.arange(0, dim, 2, dtype=torch.float64) / dim)[None, :]
    return ops.RotaryTables(torch.cos(angle).float().to(DEV).contiguous(), torch.sin(angle).float().to(DEV).contiguous(), dim, layout)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d, dv, n_q, n_kv", [(16, 16, 2, 1), (64, 64, 4, 2), (24, 10, 4, 2), (18, 26, 3, 1), (128, 32, 6, 1),
                                              (128, 128, 8, 2), (48, 48, 3, 3), (96, 96, 16, 1)])
@pytest.mark.parametrize("sink", [None, 2.0, -1.0])
def test_one_loud_key_among_hundreds_and_the_sink_against_the_closed_form(dtype, d, dv, n_q, n_kv, sink):
    """300 keys of which one is loud, in ten places (the first token, either side of a page border, far
    back, the query's own), as one prompt and with the second half decoded token by token: the
    output is the closed form of the softmax with the sink's term in the denominator, and a sink
    left out, scaled, or counted per key would not be."""
    from thing_htn_2026_b200 import ops
    T, t, scale = 300, TORCH[dtype], 0.5
    sinks = None if sink is None else (torch.full((n_q,), sink) + torch.arange(n_q) * 0.25)
    for case, loud in enumerate([0, 1, 63, 64, 65, 127, 128, 200, 298, 299]):
        g = torch.Generator().manual_seed(31 * case + d)
        q = torch.randn(T, n_q, d, generator=g) * 0.3
        k = torch.randn(T, n_kv, d, generator=g) * 0.3
        v = torch.randn(T, n_kv, dv, generator=g)
        k[loud] = q[T - 1].reshape(n_kv, n_q // n_kv, d)[:, 0] * 8.0        # loud for the last row's first head of each group
        q, k, v = q.to(t), k.to(t), v.to(t)
        proj = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], dim=1).to(DEV).contiguous()
        for first in (T, T // 2):
            kv = KeysAndValues(n_kv, d, dv, dtype)
            outs, at = [], 0
            for count in [first] + [1] * (T - first):
                rows = kv.rows(count)
                view = kv.cache.kv_view(0)
                qq = ops.qk_prepare(proj[at:at + count].contiguous(), None, None, None, 1.0, None, rows, view, n_q, False, True, kv.err)
                tiles, size = None, ops.prompt_attention_tile(t, d, 64, n_q, n_kv, dv) if count > 1 else 0
                if size:        # keys and values of one size that the tensor-core prompt kernel takes
                    row0, n_rows = ops.row_tiles_of([count], [at], size)
                    as_dev = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
                    tiles = ops.RowTiles(as_dev(row0), as_dev(n_rows), len(row0), size)
                outs.append(ops.attention(qq, rows, view, n_q, scale, None, kv.err, tiles, exact_weights=True,
                                          sinks=None if sinks is None else sinks.to(DEV)))
                kv.done(count)
                at += count
            got = torch.cat(outs).float().cpu().view(T, n_q, dv)
            qf, kf, vf = q.double(), k.double(), v.double()
            for head in range(n_q):
                group = head // (n_q // n_kv)
                s = (qf[:, head] @ kf[:, group].t()) * scale
                s = s.masked_fill(torch.arange(T)[None, :] > torch.arange(T)[:, None], -math.inf)
                e = torch.exp(s - s.max(-1, keepdim=True).values)
                extra = 0.0 if sinks is None else torch.exp(sinks[head].double() - s.max(-1, keepdim=True).values)
                want = (e / (e.sum(-1, keepdim=True) + extra)) @ vf[:, group]
                tol = 2e-5 if dtype == "float32" else 2e-2
                assert (got[:, head].double() - want).abs().max() <= tol * max(1.0, want.abs().max().item()), (loud, first, head)
                if sinks is not None and head == 0:
                    without = (e / e.sum(-1, keepdim=True)) @ vf[:, group]
                    assert (without - want).abs().max() > 0.02          # the comparison would see a sink left out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("dv, layout", [(10, "half"), (32, "half"), (12, "interleaved"), (64, "half")])
def test_values_turned_by_their_place_come_back_turned_by_the_distance(dtype, dv, layout):
    """One key takes all the weight; the read-out, turned back at the reader, is the key's value
    turned by (its place - the reader's), at distances across page borders and far back, in a prompt
    and decoded; the gate's logit is large, so the gate is one."""
    from thing_htn_2026_b200 import ops
    T, t, d, base = 260, TORCH[dtype], 8, 50.0
    tables = rope_tables(dv, base, layout)
    for loud in (0, 63, 64, 200, 259):
        g = torch.Generator().manual_seed(loud)
        q = torch.zeros(T, 1, d)
        q[:, 0, 0] = 1.0
        k = torch.zeros(T, 1, d)
        k[loud, 0, 0] = 60.0
        v = torch.randn(T, 1, dv, generator=g)
        gate = torch.full((T, dv), 30.0)
        proj = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1), gate], dim=1).to(t).to(DEV).contiguous()
        for first in (T, 100):
            kv = KeysAndValues(1, d, dv, dtype)
            outs, at = [], 0
            for count in [first] + [1] * (T - first):
                rows = kv.rows(count)
                view = kv.cache.kv_view(0)
                piece = proj[at:at + count].contiguous()
                qq = ops.qk_prepare(piece, None, None, None, 1.0, None, rows, view, 1, False, True, kv.err, value_rotary=tables)
                a = ops.attention(qq, rows, view, 1, 1.0, None, kv.err, None, exact_weights=True)
                outs.append(ops.rotate_gate(a, piece, 2 * d + dv, 1, dv, tables, rows, kv.err, 0.5))
                kv.done(count)
                at += count
            got = torch.cat(outs).float().cpu()
            vv = v.to(t).double()[loud, 0]
            for row in (loud, min(T - 1, loud + 1), min(T - 1, loud + 70), T - 1):
                turn = (loud - row) * base ** (-torch.arange(0, dv, 2, dtype=torch.float64) / dv)
                c, s = torch.cos(turn), torch.sin(turn)
                if layout == "half":
                    a, b = vv[:dv // 2], vv[dv // 2:]
                    want = torch.cat([a * c - b * s, b * c + a * s])
                else:
                    a, b = vv[0::2], vv[1::2]
                    want = torch.stack([a * c - b * s, b * c + a * s], dim=1).reshape(-1)
                tol = 1e-4 if dtype == "float32" else 4e-2
                assert (got[row].double() - 0.5 * want).abs().max() <= tol * max(1.0, want.abs().max().item()), (loud, first, row)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d, e", [(6, 4), (10, 20), (64, 32), (130, 6)])
def test_linear_attention_keeps_a_far_key_by_its_decay(dtype, d, e):
    """One loud key 270 tokens back and a query that asks for it: with a decay of 1 the read-out is
    the key's value, with 0.9 it has faded by 0.9^270, with a gate per channel by the product of the
    channel's gates since; the state is carried over steps of unequal sizes, and a slot that is
    opened again starts from nothing."""
    from thing_htn_2026_b200 import ops
    from thing_htn_2026_b200.cache import SequenceCache
    from thing_htn_2026_b200.cache.sequence_cache import StateSpec
    T, t, heads, loud = 300, TORCH[dtype], 3, 29
    proj = torch.zeros(T, heads * (2 * d + e))
    g = torch.Generator().manual_seed(d)
    value = torch.randn(heads, e, generator=g)
    proj[loud, heads * d:2 * heads * d] = torch.eye(d)[1].repeat(heads) * 4.0          # k: channel 1
    proj[loud, 2 * heads * d:] = value.reshape(-1)
    proj[T - 1, :heads * d] = torch.eye(d)[1].repeat(heads) * 0.5                          # q asks for channel 1
    proj = proj.to(t).to(DEV)
    z = rand((T, heads * d), 7).to(DEV).contiguous()
    bias = rand((heads * d,), 8, 2.0).add(3.0).to(DEV)
    decay = torch.tensor([1.0, 0.9, 0.0])
    for mode in ("constant", "gated"):
        cache = SequenceCache([StateSpec((heads, e, d))], max_tokens=512, dtype=t, device=DEV, max_slots=2)
        for attempt in range(2):
            (slot,) = cache.open(1)
            outs, at = [], 0
            for count in [100, 1, 1, 2, 64, 131, 1]:
                cache.prepare([slot], [count])
                cu = torch.tensor([0, count], dtype=torch.int32, device=DEV)
                slots = torch.tensor([slot], dtype=torch.int32, device=DEV)
                rows = ops.step_rows(cu, slots, cache.seq_lens, count, count)
                kwargs = dict(decay=decay.to(DEV)) if mode == "constant" else dict(gate=z[at:at + count].contiguous(), gate_bias=bias, tau=4.0)
                outs.append(ops.linear_attention(proj[at:at + count].contiguous(), (0, heads * d, 2 * heads * d),
                                                 cache.state_view(0), rows, heads, d, e, q_scale=2.0, **kwargs))
                ops.advance(cache.seq_lens, slots, cu)
                cache.commit([slot], [count])
                at += count
            got = torch.cat(outs).cpu().double()
            vt = value.to(t).double()
            if mode == "constant":
                fade = decay.double() ** (T - 1 - loud)
            else:
                a = torch.sigmoid(z.cpu().double() + bias.cpu().double()) ** 0.25
                fade = a[loud + 1:].prod(0).view(heads, d)[:, 1]
            want = fade[:, None] * vt * 4.0 * 0.5 * 2.0
            tol = 1e-4 if dtype == "float32" else 2e-2
            assert (got[T - 1] - want).abs().max() <= tol * max(1.0, want.abs().max().item()), (mode, attempt)
            assert got[:loud].abs().max() == 0.0 and got[loud + 1:T - 1].abs().max() == 0.0
            cache.close([slot])


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
    """A prompt of 40 and 190 tokens decoded one by one: states, rings and keys are carried through
    the cache step after step, over three page borders."""
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
    """Two batches, one after the other, in a cache that holds one of them: the second batch takes
    the slots and pages that the first gave back.  Every request also alone."""
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
def test_the_sum_of_the_streams_after_every_layer(models, name):
    """The float32 streams after each layer of a short prompt (what the layer hands on, with its
    pending write carried out), summed, through the model's own layers and cache."""
    from thing_htn_2026_b200 import ops
    from thing_htn_2026_b200.cache import SequenceCache
    from thing_htn_2026_b200.engine.loading import load_model
    from thing_htn_2026_b200.parts import StepContext
    toks = tiny.tokens(name, 37, 5)
    want = plain.model_forward(models[name], toks, torch.float32)[1]
    with torch.inference_mode():
        model = load_model(models[name], "float32", DEV)
        cache = SequenceCache(model.cache_needs(), max_tokens=128, dtype=torch.float32, device=DEV)
        (slot,) = cache.open(1)
        n = len(toks)
        cache.prepare([slot], [n])
        model.ensure_positions(n)
        cu = torch.tensor([0, n], dtype=torch.int32, device=DEV)
        slots = torch.tensor([slot], dtype=torch.int32, device=DEV)
        err = ops.new_error_word(DEV)
        ctx = StepContext(rows=ops.step_rows(cu, slots, cache.seq_lens, n, n, max_context=n), cache=cache, err=err, inputs={})
        h, d = model.embedding.forward(torch.tensor(toks, dtype=torch.int32, device=DEV), err, ctx.rows), None
        s = model.config.streams or 1
        for k, entry in enumerate(model.plan.schedule):
            h, d = model.layers[entry.layer].forward(h, d, ctx, entry)
            X, _ = ops.hyper_norm(h.clone(), s, torch.float32, y=d.tensor, written=d.write)
            got = X.view(n, s, -1).sum(1).cpu()
            worst = (got - want[k]).abs().max().item()
            assert worst <= 3e-5 * max(1.0, want[k].abs().max().item()), f"after layer {k}: the streams' sum differs by {worst:.3e}"
        assert int(err.item()) == 0


def test_what_the_plain_implementation_would_show(models):
    """The plain implementation moves far when positions start at 1 (rotation of keys and values),
    so the comparisons above would notice a position that is one off."""
    toks = tiny.tokens("a", 60, 77)
    right = plain.model_logits(models["a"], toks, torch.float64).numpy()
    shifted = plain.model_logits(models["a"], [toks[0]] + toks, torch.float64).numpy()[1:]
    assert position_error(right[1:], shifted[1:]).min() > 1e-3


def greedy_by_plain(folder, prompt, n_new):
    model = plain.read_model(folder)
    seq, margins = list(prompt), []
    for _ in range(n_new):
        logits = plain.model_forward(folder, seq, torch.float64, model)[0][-1]
        top = logits.topk(2).values
        margins.append(float(top[0] - top[1]))
        seq.append(int(logits.argmax()))
    return seq[len(prompt):], margins


@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("name", ["a", "c", "d"])
def test_greedy_generation_through_the_engine(models, name, graphs):
    """Engine.generate: the library's own entry point, scheduler, captured decode step and token
    choice, on prompts of unequal lengths, against greedy continuation by the plain implementation
    (up to the first step whose two best logits are closer than rounding)."""
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
