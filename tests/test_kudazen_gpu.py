"""Kudazen on the GPU against the plain implementation (``tests/plain/kudazen_plain.py``): every mechanism alone, whole
prompts against token-by-token decoding, portions down to two tokens, batches of unequal requests against each alone,
pages and state slots that are freed and taken again, keys just inside and just outside a chunk, at page borders and far
away, the sink of the softmax, the first tokens, long decoding, sizes that differ in every respect between the
configurations, layers that use another layer's tensors, and greedy generation through ``Engine.generate``.

The configurations and weights are made here.  Weights are drawn so that a fault shows: matrices of N(0, 1.5^2 / in) make the
attention peaked, sinks are large enough to take a good part of the softmax, the clamps of the feed-forward cut often, and
where a test is about one key a marker token, whose key points where the last query points, makes that key's score stand out.
float32 runs are held to 3e-4 of the largest logit, which no wrong key, chunk or lost state survives; bfloat16 runs to 5e-2
of a row's root-mean-square logit.
"""
from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from plain import kudazen_plain as plain

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
TOLERANCE = {"float32": 3e-4, "bfloat16": 5e-2}


# ------------------------------------------------------------------------------------------ configurations
def attention(heads, kv_heads, dim, vdim, scale, chunk=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if chunk is not None:
        mixer["mask"] = {"size": chunk}
    return "attention", mixer


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base=10000.0):
    return "latent_attention", {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale,
                                "rot": {"dims": rot_dim, "base": base}}


def wkv(heads, dim, decay_rank=None):
    mixer = {"heads": heads, "dim": dim}
    if decay_rank is not None:
        mixer["decay_rank"] = decay_rank  # read by the package when it makes tensors; a checkpoint's tensors decide otherwise
    return "wkv", mixer


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def layer(kind_and_mixer, mlp=None):
    return {"type": kind_and_mixer[0], "mixer": kind_and_mixer[1], "mlp": mlp}


def again(layers, index):
    """One more layer that uses the tensors of ``layers[index]``."""
    return {**layers[index], "weights_of": index}


def document(width, vocab, layers, groups, eps=1e-5):
    return {"architecture": "Kudazen", "vocab": vocab, "width": width, "norm": {"eps": eps, "groups": groups}, "layers": layers}


def _a_layers():
    layers = [layer(attention(4, 2, 24, 16, 0.3, chunk=40), dense(72, 0.8)), layer(latent(3, 12, 8, 20, 24, 16, 0.35), dense(40, 1.5)),
              layer(wkv(3, 20, 5)), layer(latent(2, 8, 16, 8, 12, 40, 0.4, base=500.0))]
    return layers + [again(layers, 0), again(layers, 2)]


def _b_layers():
    layers = [layer(wkv(5, 8, 3), dense(60, 3.0)), layer(latent(5, 24, 4, 12, 36, 20, 0.2, base=1e6)), layer(attention(6, 1, 8, 20, 0.5, chunk=7), dense(90, 0.5)),
              layer(attention(2, 2, 40, 40, 0.15))]
    return layers + [again(layers, 1), again(layers, 1), again(layers, 0)]


# Two models that differ in every size, in the order of their layers, in which layers lend their tensors, in the groups of the norm
# and in eps (A's is large enough to show where it stands: under every root, also the one of the time mixing's heads, whose output is
# near zero now and then); heads of unequal key and value size, one key/value head for six, chunks that are no multiple of a page (40, 7) and
# none at all, a rotated part smaller and larger than the plain part, latents smaller and larger than the queries' latent.
CONFIGS = {"A": document(64, 131, _a_layers(), groups=4, eps=2e-2), "B": document(96, 211, _b_layers(), groups=1, eps=1e-6)}
# One layer each: a mechanism alone (no feed-forward unless the feed-forward is what stands alone).
ALONE = {
    "attention": document(48, 97, [layer(attention(4, 2, 24, 24, 0.3, chunk=24))], groups=3),
    # heads of 64 and 128 with keys and values of one size: in bfloat16 these take the tensor-core kernels (chunks of 24 and of 100 cross
    # their key tiles of 64 anywhere)
    "attention_64": document(64, 97, [layer(attention(4, 2, 64, 64, 0.01, chunk=24))], groups=2),
    "attention_128": document(64, 61, [layer(attention(6, 2, 128, 128, 0.08, chunk=100))], groups=1),
    "attention_open": document(40, 61, [layer(attention(3, 3, 8, 12, 0.6))], groups=1),
    "latent": document(48, 97, [layer(latent(3, 12, 8, 20, 24, 24, 0.12))], groups=2),
    "latent_wide": document(40, 61, [layer(latent(1, 136, 24, 72, 200, 8, 0.1))], groups=5),
    # a record of 26 entries is no multiple of 16: in bfloat16 too this one stays in the kernel with float lanes
    "latent_odd": document(40, 61, [layer(latent(2, 10, 6, 12, 20, 16, 0.25))], groups=1),
    "wkv": document(48, 97, [layer(wkv(3, 20, 5))], groups=2),
    "wkv_wide": document(40, 61, [layer(wkv(1, 136, 2))], groups=1),
    "dense": document(48, 97, [layer(wkv(1, 4, 1), dense(100, 0.7))], groups=6),
}


def make_weights(doc: dict, seed: int, gain: float = 1.5) -> dict[str, torch.Tensor]:
    """bfloat16 tensors under the design's names: matrices N(0, gain^2 / in), norm weights and temperatures around 1, sinks around 1,
    mixing weights of the token shift over [0, 1], decays spread over their useful range."""
    from hyperion_b200.models import DecoderModel, get_architecture

    entry = get_architecture("Kudazen")
    model = DecoderModel(entry.build_spec(entry.read_config(doc)), torch.float32, torch.device("meta"))
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, wanted in model.expected_tensors().items():
        shape = tuple(wanted.shape)
        last = name.rsplit(".", 1)[-1]
        if last in ("norm", "norm1"):
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif last == "temp":
            t = 1.0 + 0.25 * torch.randn(shape, generator=g)
        elif last == "sink":
            t = 1.0 + 1.5 * torch.randn(shape, generator=g)
        elif ".mu." in name:
            t = torch.rand(shape, generator=g)
        elif last == "w0":
            t = -2.5 + 1.2 * torch.randn(shape, generator=g)
        elif last == "u":
            t = 0.6 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) * (gain / shape[-1] ** 0.5)
        out[name] = t.to(torch.bfloat16)
    # Time mixing divides a head's output by its root mean square.  On the first tokens of a sequence that output is little more than
    # (sum_i u_i k_i r_i) v, and with keys and receptances that know nothing of one another the sum crosses zero now and then: the head's
    # sign then hangs on the last bit of the rows before it, in any arithmetic.  Keys that lean towards the receptance and a positive
    # bonus keep the sum away from zero.
    for name in [n for n in out if n.endswith(".mix.w0")]:
        p = name[: -len("w0")]
        out[p + "k"] = ((out[p + "r"].float() + 0.6 * out[p + "k"].float()) / 1.36 ** 0.5).to(torch.bfloat16)
        out[p + "u"] = (0.3 + 0.6 * torch.rand(out[p + "u"].shape, generator=g)).to(torch.bfloat16)
    return out


def align_keys_with_queries(doc: dict, weights: dict[str, torch.Tensor]) -> None:
    """Make one score stand out: keys are made by the matrices that make the queries (every key head takes its first query head's
    matrix; a latent's key side takes the query side's down-projection, norm weight and plain rows), so a key made from the same
    token as the query meets it with cosine 1 where other keys' cosines are about 1 / sqrt(dim)."""
    for index, entry in enumerate(doc["layers"]):
        m, p = entry["mixer"], f"l{index}.mix."
        if entry["type"] == "attention":
            rep, d = m["heads"] // m["kv_heads"], m["dim"]
            weights[p + "k"] = weights[p + "q"].view(m["heads"], d, -1)[::rep].reshape(m["kv_heads"] * d, -1).clone()
        elif entry["type"] == "latent_attention":
            assert m["q_rank"] == m["kv_rank"]
            weights[p + "dkv"][: m["kv_rank"]] = weights[p + "dq"]
            weights[p + "dkv.norm"] = weights[p + "dq.norm"].clone()
            weights[p + "uk"] = weights[p + "uq"].view(m["heads"], m["dim"] + m["rot_dim"], -1)[:, : m["dim"]].reshape(m["heads"] * m["dim"], -1).clone()
    # the last token of the vocabulary is the marker, the one before it the query: the marker's embedding is mostly the
    # query's, so its key points where the query points, and partly its own, so its value is another
    own = torch.randn(weights["embed"].shape[1], generator=torch.Generator().manual_seed(99))
    weights["embed"][-1] = ((2.0 * weights["embed"][-2].float() + own) / 5 ** 0.5).to(torch.bfloat16)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    from hyperion_b200.weights import write_file

    root = tmp_path_factory.mktemp("kudazen_models")
    made = {}
    for index, (name, doc) in enumerate({**CONFIGS, **ALONE}.items()):
        folder = root / name
        folder.mkdir()
        (folder / "config.json").write_text(json.dumps(doc))
        # A: six layers of width 64 carry rounding further than B's seven of width 96; with matrices of 1.2 / sqrt(in) a bfloat16 run stays a
        # rounding away from the plain float64 one
        weights = make_weights(doc, 23 + index, gain=1.2 if name == "A" else 1.5)
        if name in ("attention", "attention_64", "latent"):
            align_keys_with_queries(doc, weights)
        if name in ("attention", "attention_64"):  # slopes up to 1/4 per position would bury a key 23 places back under any score
            weights["l0.mix.temp"] = torch.tensor([6.0, 5.0, 7.0, 4.0], dtype=torch.bfloat16)
        if name == "latent":  # a flat attention with large sinks and a loud output: a far key and the sink both move the logits
            weights["l0.mix.o"] = (3.0 * weights["l0.mix.o"].float()).to(torch.bfloat16)
            weights["l0.mix.sink"] = (2.0 + weights["l0.mix.sink"].float()).to(torch.bfloat16)
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


def assert_close(got: np.ndarray, want: np.ndarray, dtype: str, what=None) -> None:
    assert relative_error(got, want) <= TOLERANCE[dtype], what


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
    if name.startswith("latent"):  # which kernel runs: the tensor cores in bfloat16 when the record's size allows
        assert engine.model.layers[0].mixer.fast == (dtype == "bfloat16" and name != "latent_odd")
    assert_close(run_cut(engine, "w", ids, [len(ids)]), want, dtype, "whole")
    assert_close(run_cut(engine, "p", ids, [5, 2, 1, 9]), want, dtype, "portions")


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("part", [40, 42, 516])
@pytest.mark.parametrize("groups", [1, 2, 5])
def test_sum_of_two_sublayers_then_norm_in_groups(groups, part, out_dtype):
    """h <- h + (a + b), then every group of the row over its own root mean square, times the weight: against the plain function;
    with a choice of rows the stream stays as it was."""
    from hyperion_b200 import ops

    g = torch.Generator().manual_seed(groups)
    tokens, hidden, eps = 37, part * groups, 1e-5  # parts of a multiple of four columns take the kernel's 16-byte form
    h = torch.randn(tokens, hidden, generator=g) * 3
    a, b = torch.randn(tokens, hidden, generator=g), torch.randn(tokens, hidden, generator=g)
    a, b = (a.to(out_dtype), b.to(out_dtype))
    w = 1 + 0.3 * torch.randn(hidden, generator=g)
    total = h.double() + (a.double() + b.double())
    want = plain.group_norm(total, w.double(), groups, eps)
    stream = h.cuda()
    got = ops.add_group_rmsnorm(stream, a.cuda(), b.cuda(), w.cuda(), groups, eps, out_dtype)
    tolerance = 1e-5 if out_dtype == torch.float32 else 1e-2
    assert (got.double().cpu() - want).abs().max() <= tolerance * want.abs().max()
    assert (stream.double().cpu() - total).abs().max() <= 1e-5 * total.abs().max()
    rows = torch.tensor([36, 0, 5], dtype=torch.int32)
    kept = stream.clone()
    got = ops.add_group_rmsnorm(stream, None, None, w.cuda(), groups, eps, out_dtype, rows.cuda())
    assert torch.equal(stream, kept)
    assert (got.double().cpu() - want[rows.long()]).abs().max() <= tolerance * want.abs().max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("inter", [52, 53, 1028])
def test_clamped_gate_and_value_alone(inter, dtype):
    from hyperion_b200 import ops

    g = torch.Generator().manual_seed(4)
    x = (torch.randn(29, 2 * inter, generator=g) * 2).to(dtype)
    limit, slope = 0.9, 1.702
    gate, up = x[:, :inter].double().clamp(max=limit), x[:, inter:].double().clamp(-limit, limit)
    want = gate * torch.sigmoid(slope * gate) * (up + 1)
    got = ops.clamped_glu(x.cuda(), limit, slope)
    assert (got.double().cpu() - want).abs().max() <= (1e-6 if dtype == torch.float32 else 1e-2)
    assert (x[:, :inter] > limit).any() and (x[:, inter:] < -limit).any() and (x[:, :inter] < -limit).any()  # the gate has no lower limit: such entries were there


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
        assert_close(got, want, dtype, how)
        assert rows_over(got, results["whole"], TOLERANCE[dtype]) <= 0.03, how  # the same arithmetic on both sides


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
    assert_close(np.concatenate(got_rows), np.concatenate(want_rows), dtype)
    assert max(len(users) for users in slots_seen.values()) >= 2  # a slot served more than one request


def _marked(seed: int, length: int, vocab: int, back: int) -> list[int]:
    """Random tokens that end in the query token, with the marker ``back`` places before it and nowhere else."""
    ids = ids_for(seed, length, vocab - 2)  # the last two tokens of the vocabulary are kept for the marked places
    ids[-1], ids[-1 - back] = vocab - 2, vocab - 1
    return ids


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["attention", "attention_64"])
def test_keys_just_inside_and_just_outside_a_chunk(folders, name, dtype):
    """One attention that sees chunks of 24 positions over pages of 8: a marker token whose key scores high against the last query
    (the layer's key matrices are its query matrices) stands at a chosen place.  The query is put at the last, the first and a middle
    place of its chunk; the marker at the first place of the query's chunk (seen), the last place of the chunk before (not seen), one
    place back, a page border back.  Each case runs as a whole prompt and with the tail decoded token by token."""
    from hyperion_b200.engine.batch import StepEntry

    vocab, chunk = ALONE[name]["vocab"], 24
    engine = engine_for(folders[name], dtype, page_size=8)
    if name == "attention_64":
        assert engine.model.layers[0].mixer.fast == (dtype == "bfloat16")
    cases = []
    for length in (5 * chunk, 5 * chunk + 1, 5 * chunk + 12, 3 * chunk - 1):  # the query at place 23, 0, 11, 22 of its chunk
        inside = (length - 1) % chunk
        cases += [(length, back) for back in {inside, inside + 1, 1, 8, 16, inside - 1} if 0 < back < length]
    for length, back in sorted(set(cases)):
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
    # the marked key and the chunk's edge matter: the plain logits move by many float32 tolerances when the key is taken away, and
    # a chunk that is one place longer or shorter moves them too
    seen, unseen = _marked(1, 5 * chunk, vocab, 23), _marked(1, 4 * chunk + 4, vocab, 4)  # places 96 and 119; places 95 and 99
    without = list(seen)
    without[-1 - 23] = 0
    base = plain_logits(folders[name], seen)[-1]
    assert relative_error(plain_logits(folders[name], without)[-1], base) > 100 * TOLERANCE["float32"]
    config, weights = plain.read_model_folder(folders[name])
    for ids, size in ((seen, chunk - 1), (unseen, chunk + 1)):  # 96 leaves 119's chunk; 95 enters 99's
        other = json.loads(json.dumps(config))
        other["layers"][0]["mixer"]["mask"]["size"] = size
        assert relative_error(plain.forward(other, weights, ids).numpy()[-1], plain_logits(folders[name], ids)[-1]) > 100 * TOLERANCE["float32"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_key_far_away_among_hundreds_and_the_sink(folders, dtype):
    """Attention over latents with a sink: the marker stands 1, 7, 8, 9, 64, 300 and 690 places behind the last query among 700 tokens,
    as a whole prompt, in two portions cut between marker and query, and with the tail decoded."""
    from hyperion_b200.engine.batch import StepEntry

    name, vocab = "latent", ALONE["latent"]["vocab"]
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
    ids = _marked(801, 700, vocab, 690)
    base = plain_logits(folders[name], ids)[-1]
    without = list(ids)
    without[-1 - 690] = 0
    assert relative_error(plain_logits(folders[name], without)[-1], base) > 15 * TOLERANCE["float32"]
    config, weights = plain.read_model_folder(folders[name])  # and the sink: without it the plain logits are others
    weights["l0.mix.sink"] = torch.full_like(weights["l0.mix.sink"], -30.0)
    ids = ids_for(3, 75, vocab)
    assert relative_error(plain.forward(config, weights, ids).numpy(), plain_logits(folders[name], ids)) > 100 * TOLERANCE["float32"]


def _latent_attention_in_float(query, heads, record, value, cache, table, counts, firsts, page, scale, sinks):
    """Every token alone, in float64: its keys are the records of positions 0 .. its own, its values their first entries."""
    out, at = [], 0
    for row, (count, first) in enumerate(zip(counts, firsts)):
        context = first + count
        records = torch.cat([cache[int(table[row, j // page]), 0, j % page][None] for j in range(context)]).double()
        for i in range(count):
            q = query[at].double().view(heads, record)
            scores = (q @ records[: first + i + 1].T) * scale
            if sinks is not None:
                scores = torch.cat([scores, sinks.double()[:, None]], dim=1)
            weights = torch.softmax(scores, dim=1)[:, : first + i + 1]
            out.append((weights @ records[: first + i + 1, :value]).reshape(-1))
            at += 1
    return torch.stack(out)


@pytest.mark.parametrize("heads,record,value,page", [(3, 32, 24, 8), (16, 96, 64, 16), (5, 208, 200, 4), (32, 48, 40, 8), (1, 16, 8, 8)])
@pytest.mark.parametrize("with_sink", [False, True])
def test_latent_attention_on_tensor_cores_against_float(heads, record, value, page, with_sink):
    """The tensor-core kernel alone: rows of 1 to 70 tokens behind 0 to 300 cached ones over shuffled pages, in blocks of 16 and of 32
    rows, with the keys whole and split 2, 3 and 7 ways (more shares than some rows have key tiles), with and without sinks; one key
    far back is made to carry most of the weight of the last query."""
    from hyperion_b200.ops import attention as fast

    g = torch.Generator().manual_seed(heads * 1000 + record)
    counts, firsts = [1, 70, 3, 1, 17], [300, 0, 129, 63, 64]
    blocks = [-(-(f + c) // page) for c, f in zip(counts, firsts)]
    pages = sum(blocks) + 5
    order = torch.randperm(pages, generator=g).tolist()
    table = torch.full((len(counts), max(blocks)), -1, dtype=torch.int32)
    for row, n in enumerate(blocks):
        for b in range(n):
            table[row, b] = order.pop()
    cache = (torch.randn(pages, 1, page, record, generator=g) * 0.7).to(torch.bfloat16)
    tokens = sum(counts)
    query = torch.randn(tokens, heads * record, generator=g).to(torch.bfloat16)
    # the last row's last query points at the record of position 2 of its request, 78 places back
    far = cache[int(table[4, 2 // page]), 0, 2 % page].float()
    query[-1] = (3.0 * far / far.norm() * record ** 0.5).repeat(heads).to(torch.bfloat16)
    sinks = (torch.randn(heads, generator=g) * 2.0) if with_sink else None
    scale = 0.9 * record ** -0.5
    want = _latent_attention_in_float(query, heads, record, value, cache, table, counts, firsts, page, scale, sinks)
    starts = [0]
    for c in counts:
        starts.append(starts[-1] + c)
    positions = torch.cat([torch.arange(c, dtype=torch.int32) + f for c, f in zip(counts, firsts)])
    dev = torch.device("cuda")
    args = (query.to(dev), heads, record, value, cache.to(dev), table.to(dev), torch.tensor(starts, dtype=torch.int32, device=dev), positions.to(dev), len(counts),
            max(counts), max(c + f for c, f in zip(counts, firsts)), scale)
    sinks_dev = sinks.to(dev) if with_sink else None
    for shape in (None, (False, 1), (True, 1), (False, 2), (True, 3), (True, 7), (False, 7)):
        got = fast.attention_latent(*args, sinks=sinks_dev, shape=shape).float().cpu().double()
        error = ((got - want).norm(dim=1) / want.norm(dim=1).clamp_min(1e-3)).max().item()
        assert error < 1.5e-2, (shape, error)
    # the far key matters to the last query: without it the plain result is another
    cache[int(table[4, 2 // page]), 0, 2 % page] = 0
    other = _latent_attention_in_float(query, heads, record, value, cache, table, counts, firsts, page, scale, sinks)
    assert ((other[-1] - want[-1]).norm() / want[-1].norm()).item() > 0.3


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
    assert_close(single, want, dtype)
    assert_close(single[:8], want[:8], dtype, "the first tokens")
    assert_close(pair, want[:2], dtype)
    whole = run_cut(engine, "whole", ids, [len(ids)])
    assert rows_over(single, whole, TOLERANCE[dtype]) <= 0.03


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["attention_64", "attention_128"])
def test_chunks_in_the_tensor_core_kernels(folders, name, dtype):
    """Heads of 64 and of 128 over 450 tokens: as one prompt (tcgen05 tiles whose queries lie on both sides of a chunk's edge), in two
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


@pytest.mark.parametrize("name", ["wkv", "wkv_wide"])
def test_a_state_that_is_carried_over_a_long_row_and_many_steps(folders, name):
    """Time mixing over 900 tokens: as one prompt, and as a prompt of 3 tokens with everything after it in portions of 2 and 61; the
    token before the first of a portion comes from the state, and so does every matrix."""
    vocab = ALONE[name]["vocab"]
    ids = ids_for(13, 900, vocab)
    want = plain_logits(folders[name], ids)
    for dtype in ("float32", "bfloat16"):
        engine = engine_for(folders[name], dtype, max_tokens=2048)
        assert_close(run_cut(engine, "w", ids, [len(ids)]), want, dtype, "whole")
        assert_close(run_cut(engine, "p", ids, [3, 2, 61, 2, 2, 61]), want, dtype, "portions")


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
    for prompt, tokens in zip(prompts, got):
        logits = plain.forward(config, weights, prompt + tokens).numpy()
        for i, token in enumerate(tokens):  # on its own tokens, every choice is the plain argmax or a near tie of it
            row = logits[len(prompt) + i - 1]
            assert row.max() - row[token] <= 2 * TOLERANCE["bfloat16"] * np.abs(row).max()


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
        assert relative_error(read(step), np.stack(rows)) <= TOLERANCE[dtype], step


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
