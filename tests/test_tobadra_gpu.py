"""Tobadra on the GPU against the plain implementation (``tests/plain/tobadra_plain.py``): every mechanism alone, whole
prompts against token-by-token decoding, portions down to two tokens, batches of unequal requests against each alone,
pages and state slots that are freed and taken again, keys just inside and just outside a window, at page borders and far
away, the first tokens, long decoding, sizes that differ in every respect between the configurations, layers that use
another layer's tensors, and greedy generation through ``Engine.generate``.

The configurations and weights are made here.  Weights are drawn so that a fault shows: matrices of N(0, gain^2 / in) make the
attention peaked, the router's matrices are four times as large again so that few choices are close calls, corrections are as large as
many scores' differences so that choice and weight part ways (in the two whole models they are whole numbers that settle the choice alone), decays are spread over their useful range, and where a test is about one key a marker token, whose key points where the
last query points, makes that key's score stand out.  float32 runs are held to 3e-4 of the largest logit, which no wrong key,
window or lost state survives; bfloat16 runs to 5e-2 of a row's root-mean-square logit.
"""
from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from plain import tobadra_plain as plain

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
TOLERANCE = {"float32": 3e-4, "bfloat16": 5e-2}


# ------------------------------------------------------------------------------------------ configurations
def attention(heads, kv_heads, dim, vdim, scale, window=None, rot=None, base=10000.0):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        mixer["mask"] = {"size": window}
    if rot is not None:
        mixer["rot"] = {"dims": rot, "base": base}
    return "attention", mixer


def lightning(heads, dim, vdim, decay):
    return "lightning", {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}


def channel_delta(heads, kv_heads, dim, vdim, conv, decay_rank=None, gate_rank=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}
    if decay_rank is not None:
        mixer["decay_rank"] = decay_rank  # read by the package when it makes tensors; a checkpoint's tensors decide otherwise
    if gate_rank is not None:
        mixer["gate_rank"] = gate_rank
    return "channel_delta", mixer


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, top, scale, identity=0, groups=None, shared=None):
    router = {"experts": experts, "top": top, "scale": scale, "identity": identity}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    mlp = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared is not None:
        mlp["shared"] = {"ff": shared}
    return mlp


def layer(kind_and_mixer, mlp=None):
    return {"type": kind_and_mixer[0], "mixer": kind_and_mixer[1], "mlp": mlp}


def again(layers, index):
    """One more layer that uses the tensors of ``layers[index]``."""
    return {**layers[index], "weights_of": index}


def document(width, vocab, layers, taps, eps=1e-5, logit_scale=1.0):
    doc = {"architecture": "Tobadra", "vocab": vocab, "width": width, "norm": {"eps": eps}, "logit_scale": logit_scale, "layers": layers}
    if taps:
        doc["canon"] = {"taps": taps}
    return doc


def _a_layers():
    layers = [layer(attention(4, 2, 24, 16, 0.3, window=40, rot=8), dense(72)),
              layer(lightning(3, 12, 20, [0.7, 0.95, 0.999]), moe(24, 5, 2, 1.7, identity=1, groups=(3, 2), shared=40)),
              layer(channel_delta(4, 2, 12, 8, 3, decay_rank=5, gate_rank=7), moe(20, 3, 3, 0.8)),
              layer(attention(2, 2, 8, 12, 0.5, rot=6, base=500.0))]
    return layers + [again(layers, 0), again(layers, 2)]


def _b_layers():
    layers = [layer(channel_delta(3, 3, 20, 12, 2, decay_rank=4, gate_rank=3), dense(60)),
              layer(attention(6, 1, 16, 16, 0.25, window=7, rot=16, base=1e6), moe(28, 6, 2, 2.5, identity=2, groups=(4, 2), shared=16)),
              layer(lightning(1, 20, 28, [0.9])),
              layer(attention(3, 3, 12, 20, 0.4, window=100), moe(16, 2, 2, 1.0, identity=2, groups=(2, 2)))]
    return layers + [again(layers, 1), again(layers, 1), again(layers, 2)]


# Two models that differ in every size, in the order of their layers, in which layers lend their tensors, in the taps of the input
# convolution, in eps and in the logits' scale; heads of unequal key and value size, one key/value head for six and one per head, windows
# that are no multiple of a page (40, 7, 100) and none at all, a rotation over part of the head, over all of it and none (values then stay
# as they are), one to three experts per token, with and without identity experts, groups, a shared expert, and a layer without a feed-forward.
CONFIGS = {"A": document(64, 131, _a_layers(), taps=3, eps=2e-3, logit_scale=1.5), "B": document(96, 211, _b_layers(), taps=5, eps=1e-6, logit_scale=0.7)}
# One layer each: a mechanism alone (no feed-forward unless the feed-forward is what stands alone).
ALONE = {
    "attention": document(48, 97, [layer(attention(4, 2, 24, 24, 0.15, window=24, rot=8))], taps=2),
    # heads of 64 and 128 with keys and values of one size: in bfloat16 these take the tensor-core kernels (windows of 24 and of 100 cross
    # their key tiles anywhere)
    "attention_64": document(64, 97, [layer(attention(4, 2, 64, 64, 0.02, window=24, rot=16))], taps=4),
    "attention_128": document(64, 61, [layer(attention(6, 2, 128, 128, 0.08, window=100, rot=128))], taps=0),
    "attention_open": document(40, 61, [layer(attention(3, 3, 8, 12, 0.6, rot=4))], taps=1),
    "lightning": document(48, 97, [layer(lightning(3, 12, 20, [0.5, 0.97, 1.0]))], taps=4),
    "lightning_wide": document(40, 61, [layer(lightning(1, 132, 72, [0.99]))], taps=2),
    "channel_delta": document(48, 97, [layer(channel_delta(4, 2, 12, 20, 4, decay_rank=6, gate_rank=5))], taps=3),
    "channel_delta_wide": document(40, 61, [layer(channel_delta(1, 1, 132, 24, 1, decay_rank=3, gate_rank=2))], taps=2),
    # (a state of 8 x 8: with fewer entries a head's output is a sum of so few products that it cancels now and then, and the norms after it
    # blow a rounding up into a difference)
    "dense": document(48, 97, [layer(lightning(2, 8, 8, [0.5, 0.9]), dense(100))], taps=2),
    "experts": document(48, 97, [layer(lightning(2, 8, 8, [0.5, 0.9]), moe(36, 6, 3, 2.0, identity=2, groups=(4, 3), shared=24))], taps=2),
    "experts_plain": document(40, 61, [layer(lightning(2, 8, 8, [0.5, 0.9]), moe(20, 5, 2, 1.0))], taps=2),
    # one expert per token out of one group: a choice that flips swaps the whole feed-forward, so this one stands alone
    "experts_one": document(40, 61, [layer(lightning(2, 8, 8, [0.5, 0.9]), moe(12, 4, 1, 2.5, identity=2, groups=(3, 1)))], taps=2),
}


def make_weights(doc: dict, seed: int, gain: float = 1.5, decided: bool = False) -> dict[str, torch.Tensor]:
    """bfloat16 tensors under the design's names: matrices N(0, gain^2 / in), norm weights around 1, biases and the router's correction
    of the size of what they are added to, decay rates spread over their useful range.  ``decided``: the corrections are even whole numbers, all
    different, so that they alone settle which experts are chosen (scores lie between 0 and 1) while the weights still follow the scores: a
    model of several layers in bfloat16 then sends every token where exact arithmetic sends it, and can be held to it row by row."""
    from hyperion_b200.models import DecoderModel, get_architecture

    entry = get_architecture("Tobadra")
    model = DecoderModel(entry.build_spec(entry.read_config(doc)), torch.float32, torch.device("meta"))
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, wanted in model.expected_tensors().items():
        shape = tuple(wanted.shape)
        last = name.rsplit(".", 1)[-1]
        if last in ("norm", "norm1", "norm2", "norm1b", "norm2b"):
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif last == "correction" and decided:
            t = 2.0 * torch.randperm(shape[0], generator=g).float()  # steps of two: a score of exactly one beside one of zero is no tie
        elif last == "correction":
            t = 0.15 * torch.randn(shape, generator=g)
        elif last == "router":  # decided scores: few tokens whose best experts lie so close that a rounding upstream swaps them
            t = torch.randn(shape, generator=g) * (4.0 * gain / shape[-1] ** 0.5)
        elif last == "A_log":
            t = -1.0 + torch.randn(shape, generator=g)
        elif last == "dt_bias":
            t = -1.0 + 1.5 * torch.randn(shape, generator=g)
        elif last == "b" and len(shape) == 1:
            t = 0.5 * torch.randn(shape, generator=g)
        elif last in ("conv", "canon1"):
            t = torch.randn(shape, generator=g) * (0.8 / shape[-1] ** 0.5)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) * (gain / shape[-1] ** 0.5)
        out[name] = t.to(torch.bfloat16)
    return out


def align_keys_with_queries(doc: dict, weights: dict[str, torch.Tensor]) -> None:
    """Make one score stand out: keys are made by the matrices and biases that make the queries (every key head takes its first query
    head's), so a key made from the same token as the query meets it with cosine 1 in the part of the head that is not rotated, where
    other keys' cosines are about 1 / sqrt(dim)."""
    for index, entry in enumerate(doc["layers"]):
        m, p = entry["mixer"], f"l{index}.mix."
        if entry["type"] == "attention":
            rep, d = m["heads"] // m["kv_heads"], m["dim"]
            weights[p + "k"] = weights[p + "q"].view(m["heads"], d, -1)[::rep].reshape(m["kv_heads"] * d, -1).clone()
            weights[p + "k.b"] = weights[p + "q.b"].view(m["heads"], d)[::rep].reshape(-1).clone()
    # the last token of the vocabulary is the marker, the one before it the query: the marker's embedding is mostly the
    # query's, so its key points where the query points, and partly its own, so its value is another
    own = torch.randn(weights["embed"].shape[1], generator=torch.Generator().manual_seed(99))
    weights["embed"][-1] = ((2.0 * weights["embed"][-2].float() + own) / 5 ** 0.5).to(torch.bfloat16)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    from hyperion_b200.weights import write_file

    root = tmp_path_factory.mktemp("tobadra_models")
    made = {}
    for index, (name, doc) in enumerate({**CONFIGS, **ALONE}.items()):
        folder = root / name
        folder.mkdir()
        (folder / "config.json").write_text(json.dumps(doc))
        weights = make_weights(doc, 23 + index, gain=1.2 if name in CONFIGS else 1.5, decided=name in CONFIGS)
        if name in ("attention", "attention_64"):
            align_keys_with_queries(doc, weights)
            # the marker's pull must not be averaged away by what the convolution adds from the tokens before
            weights["l0.canon1"] = (0.3 * weights["l0.canon1"].float()).to(torch.bfloat16)
        write_file(folder / "model.safetensors", weights)
        made[name] = folder
    return made


_plain_cache: dict = {}


def plain_logits(folder: Path, ids) -> np.ndarray:
    key = (str(folder), tuple(ids))
    if key not in _plain_cache:
        config, weights = plain.read_model_folder(folder)
        _plain_cache[key] = plain.forward(config, weights, list(ids)).numpy()
    return _plain_cache[key]


def ids_for(seed: int, count: int, vocab: int) -> list[int]:
    return torch.randint(0, vocab, (count,), generator=torch.Generator().manual_seed(seed)).tolist()


def engine_for(folder, dtype, **options):
    from hyperion_b200.api import Engine

    options.setdefault("page_size", 16)
    options.setdefault("max_tokens", 1024)
    options.setdefault("max_requests", 4)
    return Engine.from_folder(folder, dtype=dtype, **options)


def relative_error(got: np.ndarray, want: np.ndarray) -> float:
    """The largest difference against the largest logit: the sharp measure, which a float32 run meets.  For bfloat16
    results, where rounding of a peaked attention's scores moves single logits, the worst row's root-mean-square
    difference against its root-mean-square logit."""
    sharp = float(np.abs(got - want).max() / np.abs(want).max())
    if sharp <= TOLERANCE["float32"]:
        return sharp
    got, want = np.atleast_2d(got), np.atleast_2d(want)
    return float((np.sqrt(((got - want) ** 2).mean(axis=1)) / np.sqrt((want ** 2).mean(axis=1))).max())


def rows_over(got: np.ndarray, want: np.ndarray, tolerance: float) -> float:
    """The fraction of rows whose root-mean-square difference is more than ``tolerance`` of the row's root-mean-square logit."""
    got, want = np.atleast_2d(got), np.atleast_2d(want)
    return float(((np.sqrt(((got - want) ** 2).mean(axis=1)) / np.sqrt((want ** 2).mean(axis=1))) > tolerance).mean())


def has_experts(doc: dict) -> bool:
    return any(entry["mlp"] is not None and entry["mlp"]["kind"] == "moe" for entry in doc["layers"])


def assert_close(got: np.ndarray, want: np.ndarray, dtype: str, what=None, routed: bool = False, deep: bool = False) -> None:
    """``routed`` (a layer whose router follows its input): in bfloat16 a token whose best experts lie close together may go to another
    expert than in exact arithmetic, and what it then writes into a recurrence's state stays with the tokens after it: up to a fifth of the
    rows may be off.  ``deep`` (a model of several layers, its routers decided by their corrections): roundings pass through six or seven
    layers whose norms blow up what a small sublayer output carries: three rows in a hundred may be off.  Either way the middle row stays
    within half the tolerance (a fault of a kernel, a cache or a state moves every row).  float32 is held to its line without exceptions."""
    if (routed or deep) and dtype == "bfloat16":
        got2, want2 = np.atleast_2d(got), np.atleast_2d(want)
        errors = np.sqrt(((got2 - want2) ** 2).mean(axis=1)) / np.sqrt((want2 ** 2).mean(axis=1))
        over, middle = float((errors > TOLERANCE[dtype]).mean()), float(np.median(errors))
        assert over <= (0.2 if routed else 0.03) and middle <= TOLERANCE[dtype] / 2, (what, over, middle)
        return
    error = relative_error(got, want)
    assert error <= TOLERANCE[dtype], (what, error)


def run_cut(engine, name, ids, sizes) -> np.ndarray:
    """One request in portions of the given sizes (cycled), every position's logits."""
    from hyperion_b200.engine.batch import StepEntry

    rows, at, k = [], 0, 0
    while at < len(ids):
        n = min(sizes[k % len(sizes)], len(ids) - at)
        k += 1
        rows.append(engine.step([StepEntry(name, ids[at:at + n], list(range(n)))]).cpu().numpy().copy())
        at += n
    engine.finish(name)
    engine.check()
    return np.concatenate(rows)


# ------------------------------------------------------------------------------------------ every mechanism alone
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ALONE))
def test_one_layer_of_each_kind(folders, name, dtype):
    """A model of one layer: the whole prompt at once, and again in portions of 5, 2, 1, 9 tokens."""
    vocab = ALONE[name]["vocab"]
    ids = ids_for(3, 75, vocab)
    want = plain_logits(folders[name], ids)
    engine = engine_for(folders[name], dtype, page_size=8)
    routed = has_experts(ALONE[name])
    assert_close(run_cut(engine, "w", ids, [len(ids)]), want, dtype, "whole", routed)
    assert_close(run_cut(engine, "p", ids, [5, 2, 1, 9]), want, dtype, "portions", routed)


def test_router_scores_correction_groups_and_identity_choices():
    """The router alone against the plain function: softmax scores, the choice by score + correction inside the best groups, weights
    from the plain scores; also without groups, with one group kept, and with every output kept."""
    from hyperion_b200.ops import moe as ops_moe

    g = torch.Generator().manual_seed(11)
    for outputs, top, groups, scale in ((12, 4, (4, 3), 2.5), (8, 2, None, 1.0), (10, 2, (5, 1), 0.5), (6, 6, (3, 3), 1.3), (33, 5, (11, 4), 1.0)):
        hidden, tokens = 40, 57
        x = torch.randn(tokens, hidden, generator=g)
        w = {"router": torch.randn(outputs, hidden, generator=g) * 0.4, "correction": 0.2 * torch.randn(outputs, generator=g)}
        r = {"top": top, "scale": scale}
        if groups is not None:
            r["groups"] = {"count": groups[0], "keep": groups[1]}
        want_chosen, want_weight = plain.route(x.double(), {k: v.double() for k, v in w.items()}, "", r)
        chosen, weight = ops_moe.route_scored(x.cuda(), w["router"].cuda(), w["correction"].cuda(), top, groups[0] if groups else 0, groups[1] if groups else 0, scale)
        assert torch.equal(chosen.cpu().long().sort(dim=1).values, want_chosen.sort(dim=1).values), (outputs, top, groups)
        order = chosen.cpu().long().argsort(dim=1)
        want_order = want_chosen.argsort(dim=1)
        assert (torch.gather(weight.cpu().double(), 1, order) - torch.gather(want_weight, 1, want_order)).abs().max() <= 1e-6 * scale
        # choice and weight part ways: somewhere an output with a smaller score was chosen over one with a larger
        scores = torch.softmax(x.double() @ w["router"].double().T, dim=-1)
        assert not torch.equal(scores.topk(top, dim=-1).indices.sort(dim=1).values, want_chosen.sort(dim=1).values) or top == outputs


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rotation_of_heads_there_and_back(dtype):
    """Heads turned by their positions, both pairings, part of the head and all of it; turned back they are what they were."""
    from hyperion_b200 import ops

    g = torch.Generator().manual_seed(5)
    tokens, heads, dim, col0 = 19, 3, 20, 7
    positions = torch.randint(0, 5000, (tokens,), generator=g, dtype=torch.int32)
    for dims, half in ((20, True), (8, True), (12, False)):
        x = torch.randn(tokens, col0 + heads * dim + 3, generator=g).to(dtype)
        freq = (torch.tensor(777.0, dtype=torch.float64) ** (-2.0 * torch.arange(dims // 2, dtype=torch.float64) / dims)).float()
        part = x[:, col0:col0 + heads * dim].double().reshape(tokens, heads, dim)
        if half:
            want = plain.turn_halves(part, positions, dims, 777.0)
        else:
            angle = positions.double()[:, None, None] * freq.double()[None, None, :]
            u, v = part[..., 0:dims:2], part[..., 1:dims:2]
            want = torch.cat([torch.stack([u * angle.cos() - v * angle.sin(), v * angle.cos() + u * angle.sin()], dim=-1).reshape(tokens, heads, dims), part[..., dims:]], dim=-1)
        turned = x.cuda()
        ops.rotate_heads_(turned, col0, heads, dim, positions.cuda(), freq.cuda(), dims, half, 1.0)
        tolerance = 2e-3 if dtype == torch.float32 else 3e-2  # float angles of up to 5,000 radians carry an error of a few 1e-4
        assert (turned[:, col0:col0 + heads * dim].double().cpu().reshape(tokens, heads, dim) - want).abs().max() <= tolerance
        assert torch.equal(turned[:, :col0].cpu(), x[:, :col0]) and torch.equal(turned[:, col0 + heads * dim:].cpu(), x[:, col0 + heads * dim:])
        ops.rotate_heads_(turned, col0, heads, dim, positions.cuda(), freq.cuda(), dims, half, -1.0)
        assert (turned.double().cpu() - x.double()).abs().max() <= (1e-5 if dtype == torch.float32 else 5e-2)


# ------------------------------------------------------------------------------------------ whole models
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_prefill_against_token_by_token_and_portions(folders, name, dtype):
    vocab = CONFIGS[name]["vocab"]
    ids = ids_for(5, 150, vocab)
    want = plain_logits(folders[name], ids)
    engine = engine_for(folders[name], dtype, page_size=8 if name == "A" else 16)
    results = {"whole": run_cut(engine, "w", ids, [len(ids)]), "single": run_cut(engine, "s", ids, [1]),
               "pairs": run_cut(engine, "p", ids, [2]), "mixed sizes": run_cut(engine, "m", ids, [7, 2, 16, 3, 33, 1, 1, 64])}
    for how, got in results.items():
        assert_close(got, want, dtype, how, deep=True)
        assert rows_over(got, results["whole"], TOLERANCE[dtype]) <= 0.1, how  # the same arithmetic on both sides
        if dtype == "float32":
            assert np.array_equal(got, results["whole"]), how  # float32: the same bits however the work is cut


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_unequal_requests_together_over_pages_and_slots_that_are_used_again(folders, name, dtype):
    """Six requests of unequal length through a cache of 3 state slots and too few pages for all: portions of some beside
    single tokens of others, a request sitting out now and then; as one ends, the next takes its slot and pages."""
    from hyperion_b200.engine.batch import StepEntry

    vocab = CONFIGS[name]["vocab"]
    lengths = [90, 41, 130, 17, 66, 101]
    requests = {f"r{i}": ids_for(50 + i, n, vocab) for i, n in enumerate(lengths)}
    want = {rid: plain_logits(folders[name], ids) for rid, ids in requests.items()}
    engine = engine_for(folders[name], dtype, page_size=16, max_tokens=3 * 144, max_requests=3)
    waiting, live, sizes, k, step = list(requests), {}, [5, 2, 19, 3, 8, 2, 30, 4], 0, 0
    slots_seen: dict[int, set] = {}
    got_rows, want_rows = [], []
    while waiting or live:
        while waiting and len(live) < 3:
            live[waiting.pop(0)] = 0
        entries = []
        for j, rid in enumerate(list(live)):
            ids, at = requests[rid], live[rid]
            if (step + j) % 5 == 4 and len(live) > 1:
                continue
            n = 1 if at >= len(ids) - 10 else min(sizes[k % len(sizes)], len(ids) - 10 - at)
            k += 1
            entries.append(StepEntry(rid, ids[at:at + n], list(range(n))))
        logits = engine.step(entries).cpu().numpy()
        row = 0
        for entry in entries:
            at = live[entry.request]
            n = len(entry.tokens)
            got_rows.append(logits[row:row + n])
            want_rows.append(want[entry.request][at:at + n])
            row += n
            live[entry.request] = at + n
            slots_seen.setdefault(engine.cache.slot(entry.request), set()).add(entry.request)
            if at + n == len(requests[entry.request]):
                engine.finish(entry.request)
                del live[entry.request]
        step += 1
    engine.check()
    engine.cache.check()
    assert_close(np.concatenate(got_rows), np.concatenate(want_rows), dtype, deep=True)
    assert max(len(users) for users in slots_seen.values()) >= 2  # a slot served more than one request


def _marked(seed: int, length: int, vocab: int, back: int) -> list[int]:
    """Random tokens that end in the query token, with the marker ``back`` places before it and nowhere else."""
    ids = ids_for(seed, length, vocab - 2)  # the last two tokens of the vocabulary are kept for the marked places
    ids[-1], ids[-1 - back] = vocab - 2, vocab - 1
    return ids


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["attention", "attention_64"])
def test_keys_just_inside_and_just_outside_the_window(folders, name, dtype):
    """One attention with a window of 24 positions over pages of 8: a marker token whose key scores high against the last query (the
    layer's key matrices are its query matrices) stands 23 places back (the last key the window keeps), 24 places back (the first it does
    not), one place, one page and two pages back, and 22 and 25; the prompts end at and around multiples of a page.  Each case runs as a
    whole prompt and with the tail decoded token by token, so that the window also passes over decoded tokens."""
    from hyperion_b200.engine.batch import StepEntry

    vocab, window = ALONE[name]["vocab"], 24
    engine = engine_for(folders[name], dtype, page_size=8)
    if name == "attention_64":
        assert engine.model.layers[0].mixer.inner.inner.fast == (dtype == "bfloat16")
    for length in (120, 121, 127, 71):
        for back in (1, 8, 16, window - 2, window - 1, window, window + 1):
            ids = _marked(700 + length + back, length, vocab, back)
            want = plain_logits(folders[name], ids)
            whole = engine.step([StepEntry("w", ids, [len(ids) - 1])]).cpu().numpy()[0]
            engine.finish("w")
            assert relative_error(whole, want[-1]) <= TOLERANCE[dtype], (length, back)
            head = len(ids) - 30
            engine.step([StepEntry("d", ids[:head], [])])
            for at in range(head, len(ids)):
                last = engine.step([StepEntry("d", [ids[at]], [0])]).cpu().numpy()[0]
                assert relative_error(last, want[at]) <= TOLERANCE[dtype], (length, back, at)
            engine.finish("d")
    engine.check()
    # the marked key and the window's edge matter: the plain logits move by many float32 tolerances when the key is taken away, and
    # a window that is one place longer or shorter moves them too
    seen, unseen = _marked(1, 120, vocab, window - 1), _marked(1, 120, vocab, window)
    without = list(seen)
    without[-1 - (window - 1)] = 0
    base = plain_logits(folders[name], seen)[-1]
    assert relative_error(plain_logits(folders[name], without)[-1], base) > 100 * TOLERANCE["float32"]
    config, weights = plain.read_model_folder(folders[name])
    for ids, size in ((seen, window - 1), (unseen, window + 1)):  # the key 23 back leaves a window of 23; the key 24 back enters one of 25
        other = json.loads(json.dumps(config))
        other["layers"][0]["mixer"]["mask"]["size"] = size
        assert relative_error(plain.forward(other, weights, ids).numpy()[-1], plain_logits(folders[name], ids)[-1]) > 100 * TOLERANCE["float32"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_key_far_away_among_hundreds_and_rotated_values(folders, dtype):
    """An attention without a window: the marker stands 1, 7, 8, 9, 64, 300 and 690 places behind the last query among 700 tokens, as a
    whole prompt, in two portions cut between marker and query, and with the tail decoded.  What the query takes from the marker is its
    value turned by the distance between them; without that rotation the plain logits are others."""
    from hyperion_b200.engine.batch import StepEntry

    name, vocab = "attention_open", ALONE["attention_open"]["vocab"]
    engine = engine_for(folders[name], dtype, page_size=8, max_tokens=1536)
    for back in (1, 7, 8, 9, 64, 300, 690):
        ids = _marked(800 + back, 700, vocab, back)
        want = plain_logits(folders[name], ids)
        whole = engine.step([StepEntry("w", ids, [len(ids) - 1])]).cpu().numpy()[0]
        engine.finish("w")
        assert relative_error(whole, want[-1]) <= TOLERANCE[dtype], back
        cut = len(ids) - 1 - back // 2
        engine.step([StepEntry("p", ids[:cut], [])])
        last = engine.step([StepEntry("p", ids[cut:], [len(ids) - cut - 1])]).cpu().numpy()[0]
        engine.finish("p")
        assert relative_error(last, want[-1]) <= TOLERANCE[dtype], (back, "two portions")
        engine.step([StepEntry("d", ids[:-20], [])])
        for at in range(len(ids) - 20, len(ids)):
            last = engine.step([StepEntry("d", [ids[at]], [0])]).cpu().numpy()[0]
            assert relative_error(last, want[at]) <= TOLERANCE[dtype], (back, at)
        engine.finish("d")
    engine.check()
    config, weights = plain.read_model_folder(folders[name])
    ids = ids_for(3, 75, vocab)
    turned = plain.forward(config, weights, ids).numpy()

    def values_stay(x, positions, dims, base, sign=1.0, original=plain.turn_halves):
        return x if dims == config["layers"][0]["mixer"]["vdim"] else original(x, positions, dims, base, sign)

    plain.turn_halves, kept = values_stay, plain.turn_halves
    try:
        assert relative_error(plain.forward(config, weights, ids).numpy(), turned) > 100 * TOLERANCE["float32"]
    finally:
        plain.turn_halves = kept


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_first_tokens_and_long_decoding(folders, name, dtype):
    from hyperion_b200.engine.batch import StepEntry

    vocab = CONFIGS[name]["vocab"]
    ids = ids_for(8, 400, vocab)
    want = plain_logits(folders[name], ids)
    engine = engine_for(folders[name], dtype, page_size=32, max_tokens=512)
    rows = []
    for at, token in enumerate(ids):  # position 0 alone, then every other one: a one-token prompt and 399 decoded tokens
        rows.append(engine.step([StepEntry("r", [token], [0])]).cpu().numpy()[0].copy())
    engine.finish("r")
    pair = engine.step([StepEntry("pair", ids[:2], [0, 1])]).cpu().numpy().copy()
    engine.finish("pair")
    engine.check()
    single = np.stack(rows)
    assert_close(single, want, dtype, deep=True)
    assert_close(single[:8], want[:8], dtype, "the first tokens")
    assert_close(pair, want[:2], dtype)
    whole = run_cut(engine, "whole", ids, [len(ids)])
    assert rows_over(single, whole, TOLERANCE[dtype]) <= 0.1


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["attention_64", "attention_128"])
def test_windows_in_the_tensor_core_kernels(folders, name, dtype):
    """Heads of 64 and of 128 over 450 tokens: as one prompt (tiles whose queries' windows begin in the middle of a key tile), in two
    portions and a tail decoded token by token (the split-key kernel), and three requests of unequal progress side by side."""
    from hyperion_b200.engine.batch import StepEntry

    vocab = ALONE[name]["vocab"]
    ids = ids_for(77, 450, vocab)
    want = plain_logits(folders[name], ids)
    engine = engine_for(folders[name], dtype, max_tokens=2048)
    assert_close(run_cut(engine, "w", ids, [len(ids)]), want, dtype, "whole")
    got = [engine.step([StepEntry("d", ids[:300], list(range(300)))]).cpu().numpy().copy()]
    got.append(engine.step([StepEntry("d", ids[300:420], list(range(120)))]).cpu().numpy().copy())
    for at in range(420, 450):
        got.append(engine.step([StepEntry("d", [ids[at]], [0])]).cpu().numpy().copy())
    engine.finish("d")
    assert_close(np.concatenate(got), want, dtype, "two portions and a decoded tail")
    engine.step([StepEntry("a", ids[:199], []), StepEntry("b", ids[:30], [])])
    got = engine.step([StepEntry("a", [ids[199]], [0]), StepEntry("b", ids[30:330], list(range(300))), StepEntry("c", ids[:2], [0, 1])]).cpu().numpy()
    engine.check()
    assert_close(got, np.concatenate([want[199:200], want[30:330], want[:2]]), dtype, "side by side")


@pytest.mark.parametrize("name", ["lightning", "lightning_wide", "channel_delta", "channel_delta_wide"])
def test_a_state_that_is_carried_over_a_long_row_and_many_steps(folders, name):
    """A recurrence over 900 tokens: as one prompt (in bfloat16 a long row of a constant decay is walked in segments), and as a prompt of
    3 tokens with everything after it in portions of 2 and 61; every matrix and the convolutions' last inputs come from the state."""
    vocab = ALONE[name]["vocab"]
    ids = ids_for(13, 900, vocab)
    want = plain_logits(folders[name], ids)
    for dtype in ("float32", "bfloat16"):
        engine = engine_for(folders[name], dtype, max_tokens=2048)
        assert_close(run_cut(engine, "w", ids, [len(ids)]), want, dtype, "whole")
        assert_close(run_cut(engine, "p", ids, [3, 2, 61, 2, 2, 61]), want, dtype, "portions")


def test_the_input_convolution_reads_the_rows_before_the_portion(folders):
    """Five taps: the first four tokens of every portion read rows of the portion before, the first four of a request read zeros.  A
    request that takes a slot another has left must not read what that one kept."""
    from hyperion_b200.engine.batch import StepEntry

    name, vocab = "B", CONFIGS["B"]["vocab"]
    first, second = ids_for(31, 40, vocab), ids_for(32, 40, vocab)
    engine = engine_for(folders[name], "float32", max_requests=1)
    assert np.array_equal(run_cut(engine, "x", first, [1, 2, 3, 4, 5, 25]), run_cut(engine, "y", first, [40]))
    got = run_cut(engine, "z", second, [3, 37])  # the slot that held x and y
    assert relative_error(got, plain_logits(folders[name], second)) <= TOLERANCE["float32"]
    config, weights = plain.read_model_folder(folders[name])
    for key in [k for k in weights if k.endswith("canon1")]:
        weights[key] = torch.zeros_like(weights[key])
    assert relative_error(plain.forward(config, weights, second).numpy(), plain_logits(folders[name], second)) > 100 * TOLERANCE["float32"]


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_greedy_generation_through_the_scheduler(folders, name):
    from hyperion_b200.sampling import SamplingParams

    vocab = CONFIGS[name]["vocab"]
    prompts = [ids_for(300 + i, n, vocab) for i, n in enumerate([5, 37, 1, 80, 23])]
    config, weights = plain.read_model_folder(folders[name])

    def greedy(prompt, count):
        ids = list(prompt)
        for _ in range(count):
            ids.append(int(plain.forward(config, weights, ids)[-1].argmax()))
        return ids[len(prompt):]

    want = [greedy(prompt, 6) for prompt in prompts]
    engine = engine_for(folders[name], "float32", max_tokens=3 * 128, max_requests=3)
    got = engine.generate(prompts, SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True), max_batch_tokens=48, prefill_chunk_busy=16)
    assert got == want
    engine = engine_for(folders[name], "bfloat16", max_tokens=3 * 128, max_requests=3)
    got = engine.generate(prompts, SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True), max_batch_tokens=48, prefill_chunk_busy=16)
    assert all(len(tokens) == 6 for tokens in got)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_through_the_command(folders, dtype, tmp_path):
    """bin/trace_run on a model of this design: two requests side by side, one ends, a third takes its place."""
    name, vocab = "A", CONFIGS["A"]["vocab"]
    a, b, c = ids_for(1, 70, vocab), ids_for(2, 33, vocab), ids_for(3, 50, vocab)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:40], "want": [39]}, {"id": "b", "tokens": b[:31], "want": [0, 30]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[40:42], "want": [0, 1]}, {"id": "b", "tokens": b[31:32], "want": [0]}], "end": []},
             {"step": 2, "entries": [{"id": "b", "tokens": b[32:], "want": [0]}], "end": ["b"]},
             {"step": 3, "entries": [{"id": "c", "tokens": c, "want": [49]}, {"id": "a", "tokens": a[42:], "want": [27]}], "end": ["a", "c"]}]
    text = "".join(json.dumps(s) + "\n" for s in steps)
    done = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folders[name]), "--dtype", dtype, "--out", str(tmp_path),
                           "--max-tokens", "192"], input=text, capture_output=True, text=True, timeout=900)
    assert done.returncode == 0, done.stderr[-3000:]
    assert [line for line in done.stdout.splitlines() if line.startswith("done ")] == [f"done {i}" for i in range(4)]
    ref = {"a": plain_logits(folders[name], a), "b": plain_logits(folders[name], b), "c": plain_logits(folders[name], c)}
    read = lambda step: np.fromfile(tmp_path / f"{step}.f32", dtype="<f4").reshape(-1, vocab)
    expected = {0: [ref["a"][39], ref["b"][0], ref["b"][30]], 1: [ref["a"][40], ref["a"][41], ref["b"][31]], 2: [ref["b"][32]],
                3: [ref["c"][49], ref["a"][69]]}
    for step, rows in expected.items():
        assert_close(read(step), np.stack(rows), dtype, step)


def test_the_command_line_writes_a_random_model_and_generates_with_it(tmp_path):
    """``python -m hyperion_b200 random`` from a config.json of this design, then ``generate`` on the folder it wrote:
    the tokens are the plain implementation's greedy ones."""
    config = tmp_path / "config.json"
    config.write_text(json.dumps(CONFIGS["B"]))
    folder = tmp_path / "model"
    run = lambda *args: subprocess.run([sys.executable, "-m", "hyperion_b200", *args], capture_output=True, text=True, timeout=900, cwd=ROOT)
    done = run("random", "--config", str(config), "--out", str(folder), "--seed", "5", "--std", "0.3")
    assert done.returncode == 0, done.stderr[-2000:]
    prompt = ids_for(71, 19, CONFIGS["B"]["vocab"])
    done = run("generate", "-m", str(folder), "--dtype", "float32", "--prompt-ids", ",".join(map(str, prompt)), "--max-tokens", "5", "--temperature", "0",
               "--ignore-eos", "--max-batch", "2")
    assert done.returncode == 0, done.stderr[-2000:]
    got = json.loads(done.stdout.strip().splitlines()[-1])
    plain_config, weights = plain.read_model_folder(folder)
    ids = list(prompt)
    for _ in range(5):
        ids.append(int(plain.forward(plain_config, weights, ids)[-1].argmax()))
    assert got["tokens"] == ids[len(prompt):] and got["finish_reason"] == "length"


# ------------------------------------------------------------------------------------------ configurations drawn at random
def _random_document(seed: int) -> dict:
    """A model whose every size, option and constant is drawn: widths, heads and groupings, head sizes that the tensor-core kernels take and
    others, windows, rotations, taps, experts with or without identities, groups and a shared expert, layers without a feed-forward, layers
    that borrow tensors, in any order."""
    import random

    r = random.Random(seed)
    width = r.choice([32, 40, 56, 64, 80, 128])

    def feed_forward():
        kind = r.choice(["none", "dense", "moe", "moe"])
        if kind == "none":
            return None
        if kind == "dense":
            return dense(r.choice([24, 50, 96]))
        experts, identity = r.randint(1, 7), r.randint(0, 3)
        outputs = experts + identity
        count = r.choice([c for c in range(1, outputs + 1) if outputs % c == 0])
        keep = r.randint(1, count)
        top = r.randint(1, min(4, keep * (outputs // count)))
        groups = (count, keep) if r.random() < 0.8 else None
        if groups is None:
            top = r.randint(1, min(4, outputs))
        return moe(r.choice([8, 20, 40]), experts, top, r.choice([0.5, 1.0, 2.5]), identity=identity, groups=groups, shared=r.choice([None, 16, 24]))

    def mixer():
        kind = r.choice(["attention", "attention", "lightning", "channel_delta"])
        if kind == "attention":
            kv = r.choice([1, 2, 3])
            heads = kv * r.choice([1, 2, 3])
            dim = r.choice([8, 16, 24, 32, 40, 64])
            vdim = r.choice([dim, dim, 12, 20, 32])
            rot = r.choice([None, dim, r.randrange(2, dim + 1, 2)])
            return attention(heads, kv, dim, vdim, r.choice([0.1, 0.2, dim ** -0.5]), window=r.choice([None, r.randint(2, 70)]), rot=rot, base=r.choice([100.0, 10000.0, 1e6]))
        if kind == "lightning":
            heads = r.randint(1, 3)
            return lightning(heads, r.choice([8, 12, 32]), r.choice([8, 20, 32]), [r.choice([0.5, 0.9, 0.99, 1.0]) for _ in range(heads)])
        kv = r.choice([1, 2])
        return channel_delta(kv * r.choice([1, 2]), kv, r.choice([8, 12, 32]), r.choice([8, 20]), r.randint(1, 4), decay_rank=r.randint(1, 6), gate_rank=r.randint(1, 6))

    layers = [layer(mixer(), feed_forward()) for _ in range(r.randint(2, 4))]
    for _ in range(r.randint(0, 2)):
        layers.insert(r.randint(1, len(layers)), None)  # a place for a layer that borrows
    filled = []  # a borrowing layer may stand before or after the layer it borrows from
    for i, entry in enumerate(layers):
        if entry is None:
            source = r.choice([j for j in range(len(layers)) if layers[j] is not None])
            filled.append({**layers[source], "weights_of": source})
        else:
            filled.append(entry)
    return document(width, r.randint(40, 300), filled, taps=r.choice([0, 1, 2, 4, 5]), eps=r.choice([1e-6, 1e-5, 1e-3]), logit_scale=r.choice([0.5, 1.0, 3.0]))


@pytest.mark.parametrize("seed", range(8))
def test_configurations_drawn_at_random(seed, tmp_path):
    """Eight models drawn at random, in float32 against the plain implementation: a whole prompt, the same in portions, and two requests of
    unequal progress side by side; in bfloat16 the middle row of the whole prompt."""
    from hyperion_b200.engine.batch import StepEntry
    from hyperion_b200.weights import write_file

    doc = _random_document(seed)
    folder = tmp_path / "model"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(doc))
    write_file(folder / "model.safetensors", make_weights(doc, 100 + seed, gain=1.2, decided=True))
    ids, other = ids_for(seed, 90, doc["vocab"]), ids_for(seed + 50, 37, doc["vocab"])
    want, want_other = plain_logits(folder, ids), plain_logits(folder, other)
    engine = engine_for(folder, "float32", page_size=8, max_tokens=512)
    assert_close(run_cut(engine, "w", ids, [len(ids)]), want, "float32", ("whole", doc))
    assert_close(run_cut(engine, "p", ids, [3, 1, 2, 17]), want, "float32", ("portions", doc))
    engine.step([StepEntry("a", ids[:61], []), StepEntry("b", other[:5], [])])
    got = engine.step([StepEntry("a", [ids[61]], [0]), StepEntry("b", other[5:], list(range(32)))]).cpu().numpy()
    engine.check()
    assert_close(got, np.concatenate([want[61:62], want_other[5:]]), "float32", ("side by side", doc))
    engine = engine_for(folder, "bfloat16", page_size=8, max_tokens=512)
    got = run_cut(engine, "w", ids, [len(ids)])
    errors = np.sqrt(((got - want) ** 2).mean(axis=1)) / np.sqrt((want ** 2).mean(axis=1))
    assert np.median(errors) <= TOLERANCE["bfloat16"], (float(np.median(errors)), doc)


def test_sizes_of_one_and_many_groups(tmp_path):
    """Every size that can be one is one (heads, key and value sizes of one and two, a window of one position, one tap, one expert, as many
    choices as router outputs, inner sizes of one), and a router of 36 outputs in 12 groups with eight query heads on one key/value head and
    seven taps: whole, in portions and token by token, in both precisions."""
    from hyperion_b200.weights import write_file

    docs = {
        "ones": document(8, 17, [layer(attention(1, 1, 2, 2, 1.0, window=1, rot=2), moe(4, 1, 1, 1.0)),
                                 layer(lightning(1, 1, 1, [1.0]), moe(4, 1, 2, 3.0, identity=1, groups=(2, 2), shared=4)),
                                 layer(channel_delta(1, 1, 1, 1, 1, decay_rank=1, gate_rank=1), dense(1)),
                                 layer(attention(1, 1, 4, 2, 0.5, window=2, rot=2))], taps=1, eps=1e-6),
        "many": document(24, 50, [layer(attention(8, 1, 16, 16, 0.25, window=33, rot=16), moe(8, 30, 6, 2.0, identity=6, groups=(12, 5), shared=8)),
                                  layer(channel_delta(6, 3, 16, 16, 4, decay_rank=2, gate_rank=2), moe(8, 9, 8, 1.0, groups=(3, 3)))], taps=7),
    }
    for name, doc in docs.items():
        folder = tmp_path / name
        folder.mkdir()
        (folder / "config.json").write_text(json.dumps(doc))
        write_file(folder / "model.safetensors", make_weights(doc, 7, gain=1.2, decided=True))
        ids = ids_for(1, 90, doc["vocab"])
        want = plain_logits(folder, ids)
        for dtype in ("float32", "bfloat16"):
            engine = engine_for(folder, dtype, page_size=8, max_tokens=512)
            for sizes in ([len(ids)], [3, 1, 2, 17], [1]):
                assert_close(run_cut(engine, "w", ids, sizes), want, dtype, (name, sizes), deep=True)
