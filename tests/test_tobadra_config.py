"""Tobadra's configuration reader and its model as data, without a GPU: every size and constant comes from the document,
a missing or malformed key is refused by name, the document is written back as it was read, a layer that borrows tensors
becomes a schedule entry with a cache of its own, and the parts ask for the design's tensor names and for the right kinds
of cache.  The plain implementation's pieces are held to hand-made cases here too."""
from __future__ import annotations

import copy

import pytest
import torch

from hyperion_b200.config import ConfigError, TobadraConfig
from hyperion_b200.models import DecoderModel, architecture_of, get_architecture
from hyperion_b200.parts import PagedTokens, RequestState
from plain import tobadra_plain as plain

DOCUMENT = {
    "architecture": "Tobadra", "vocab": 77, "width": 40, "norm": {"eps": 1e-5}, "canon": {"taps": 3}, "logit_scale": 1.5,
    "layers": [
        {"type": "channel_delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 12, "vdim": 10, "conv": 2, "decay_rank": 5, "gate_rank": 3}, "mlp": {"kind": "dense", "ff": 60}},
        {"type": "attention", "mixer": {"heads": 6, "kv_heads": 2, "dim": 12, "vdim": 20, "scale": 0.3, "mask": {"size": 50}, "rot": {"dims": 8, "base": 777.0}},
         "mlp": {"kind": "moe", "expert": {"ff": 24}, "router": {"experts": 5, "top": 2, "scale": 2.5, "identity": 1, "groups": {"count": 3, "keep": 2}}, "shared": {"ff": 16}}},
        {"type": "lightning", "mixer": {"heads": 3, "dim": 14, "vdim": 9, "decay": [0.5, 0.9, 1.0]}, "mlp": None},
        {"type": "attention", "mixer": {"heads": 2, "kv_heads": 1, "dim": 32, "vdim": 32, "scale": 0.2},
         "mlp": {"kind": "moe", "expert": {"ff": 8}, "router": {"experts": 2, "top": 2, "scale": 1.0, "identity": 0}}},
        {"type": "attention", "mixer": {"heads": 6, "kv_heads": 2, "dim": 12, "vdim": 20, "scale": 0.3, "mask": {"size": 50}, "rot": {"dims": 8, "base": 777.0}},
         "mlp": {"kind": "moe", "expert": {"ff": 24}, "router": {"experts": 5, "top": 2, "scale": 2.5, "identity": 1, "groups": {"count": 3, "keep": 2}}, "shared": {"ff": 16}},
         "weights_of": 1},
    ],
}


def test_the_document_is_read_and_written_back():
    entry = architecture_of(DOCUMENT)
    assert entry.name == "Tobadra"
    config = entry.read_config(DOCUMENT)
    assert entry.write_config(config) == DOCUMENT
    assert (config.vocab, config.width, config.eps, config.taps, config.logit_scale) == (77, 40, 1e-5, 3, 1.5)
    d = config.layers[0].mixer
    assert (d.heads, d.kv_heads, d.dim, d.vdim, d.conv, d.decay_rank, d.gate_rank) == (4, 2, 12, 10, 2, 5, 3)
    a = config.layers[1].mixer
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.window, a.rot_dims, a.rot_base) == (6, 2, 12, 20, 0.3, 50, 8, 777.0)
    assert config.layers[2].mixer.decay == (0.5, 0.9, 1.0) and config.layers[2].mlp is None
    assert (config.layers[3].mixer.window, config.layers[3].mixer.rot_dims) == (0, 0)
    f = config.layers[1].mlp
    assert (f.ff, f.experts, f.identity, f.top, f.scale, f.group_count, f.group_keep, f.shared_ff) == (24, 5, 1, 2, 2.5, 3, 2, 16)
    assert config.layers[3].mlp.shared_ff is None and config.layers[3].mlp.group_count == 0 and config.layers[0].mlp.ff == 60
    assert [config.source_of(i) for i in range(5)] == [0, 1, 2, 3, 1]
    without = copy.deepcopy(DOCUMENT)
    del without["canon"], without["logit_scale"]
    bare = TobadraConfig.from_dict(without)
    assert bare.taps == 0 and bare.logit_scale == 1.0


@pytest.mark.parametrize("path, value, key", [
    (("vocab",), 0, "vocab"), (("width",), None, "width"), (("norm", "eps"), -1.0, "norm.eps"), (("canon", "taps"), 0, "canon.taps"),
    (("logit_scale",), -2.0, "logit_scale"), (("layers", 0, "type"), "lstm", "layers[0].type"), (("layers", 0, "mixer", "conv"), 0, "layers[0].mixer.conv"),
    (("layers", 0, "mixer", "kv_heads"), 3, "layers[0].mixer.kv_heads"), (("layers", 1, "mixer", "kv_heads"), 4, "layers[1].mixer.kv_heads"),
    (("layers", 1, "mixer", "rot", "dims"), 7, "layers[1].mixer.rot.dims"), (("layers", 1, "mixer", "rot", "dims"), 16, "layers[1].mixer.rot.dims"),
    (("layers", 1, "mixer", "mask", "size"), 0, "layers[1].mixer.mask.size"), (("layers", 1, "mixer", "scale"), None, "layers[1].mixer.scale"),
    (("layers", 2, "mixer", "decay"), [0.5, 0.9], "layers[2].mixer.decay"), (("layers", 2, "mixer", "decay"), [0.5, 0.9, 1.5], "layers[2].mixer.decay"),
    (("layers", 1, "mlp", "kind"), "sparse", "layers[1].mlp.kind"), (("layers", 1, "mlp", "router", "top"), 5, "layers[1].mlp.router.top"),
    (("layers", 1, "mlp", "router", "groups", "count"), 4, "layers[1].mlp.router.groups.count"), (("layers", 1, "mlp", "router", "groups", "keep"), 4, "layers[1].mlp.router.groups.keep"),
    (("layers", 1, "mlp", "expert"), None, "layers[1].mlp.expert"), (("layers", 1, "mlp", "router", "identity"), -1, "layers[1].mlp.router.identity"),
    (("layers", 4, "weights_of"), 4, "layers[4].weights_of"), (("layers", 4, "weights_of"), 3, "layers[4].weights_of"), (("layers", 0, "mlp", "ff"), 0, "layers[0].mlp.ff"),
])
def test_a_bad_value_is_refused_by_name(path, value, key):
    document = copy.deepcopy(DOCUMENT)
    at = document
    for step in path[:-1]:
        at = at[step]
    if value is None:
        del at[path[-1]]
    else:
        at[path[-1]] = value
    with pytest.raises(ConfigError) as refused:
        TobadraConfig.from_dict(document)
    assert refused.value.key == key


def test_the_model_as_data_asks_for_the_designs_tensors_and_caches():
    entry = get_architecture("Tobadra")
    model = DecoderModel(entry.build_spec(entry.read_config(DOCUMENT)), torch.float32, torch.device("meta"))
    wanted = {name: tuple(spec.shape) for name, spec in model.expected_tensors().items()}
    assert wanted["embed"] == (77, 40) and wanted["embed.norm"] == (40,) and "head" not in wanted and wanted["final.norm"] == (40,)
    for i in range(4):
        assert wanted[f"l{i}.canon1"] == (40, 3) and wanted[f"l{i}.rg1"] == (40, 40) and wanted[f"l{i}.rg1.b"] == (40,)
        assert wanted[f"l{i}.norm1"] == wanted[f"l{i}.norm1b"] == (40,)
    assert not any(name.startswith("l4.") for name in wanted)  # the last layer has no tensors of its own
    assert wanted["l0.mix.q"] == (24, 40) and wanted["l0.mix.k"] == (24, 40) and wanted["l0.mix.v"] == (40, 40) and wanted["l0.mix.v.conv"] == (40, 2)
    assert wanted["l0.mix.b"] == (4, 40) and wanted["l0.mix.A_log"] == (4,) and wanted["l0.mix.norm"] == (10,) and wanted["l0.mix.dt_bias"] == (48,)
    assert wanted["l0.mix.a1"] == (5, 40) and wanted["l0.mix.a2"] == (48, 5) and wanted["l0.mix.g1"] == (3, 40) and wanted["l0.mix.g2"] == (40, 3)
    assert wanted["l0.mlp.up"] == (60, 40) and wanted["l0.mlp.down"] == (40, 60) and wanted["l0.rg2"] == (40, 40) and wanted["l0.norm2b"] == (40,)
    assert wanted["l1.mix.q"] == (72, 40) and wanted["l1.mix.q.b"] == (72,) and wanted["l1.mix.k"] == (24, 40) and wanted["l1.mix.v"] == (40, 40)
    assert wanted["l1.mix.v.b"] == (40,) and wanted["l1.mix.o"] == (40, 120) and wanted["l1.mix.o.b"] == (40,)
    assert wanted["l1.mlp.router"] == (6, 40) and wanted["l1.mlp.correction"] == (6,) and wanted["l1.mlp.e4.up"] == (24, 40) and "l1.mlp.e5.up" not in wanted
    assert wanted["l1.mlp.shared.up"] == (16, 40) and wanted["l1.mlp.shared.sg"] == (1, 40) and "l1.mlp.e0.gate" not in wanted
    assert wanted["l2.mix.q"] == (42, 40) and wanted["l2.mix.v"] == (27, 40) and wanted["l2.mix.g"] == (27, 40) and wanted["l2.mix.norm"] == (27,)
    assert "l2.norm2" not in wanted and "l2.rg2" not in wanted and "l3.mlp.shared.up" not in wanted and wanted["l3.mlp.router"] == (2, 40)
    assert [run.layer for run in model.spec.schedule] == [0, 1, 2, 3, 1]
    users = dict(model.cache_users())
    assert set(users) == {(i, j) for i in range(5) for j in range(2)}  # every entry: the convolution's last rows, and the mixer's own
    assert all(users[(i, 0)] == RequestState((80,), torch.float32) for i in range(5))
    assert users[(1, 1)] == users[(4, 1)] == PagedTokens((2,), (32,), 50)  # keys of 12 and values of 20 side by side, a window of 50
    assert users[(3, 1)] == PagedTokens((2, 1), (32,), 0)  # keys and values of one size: the layout every attention of the package uses
    assert users[(2, 1)] == RequestState((3 * 9 * 16,), torch.float32)
    assert users[(0, 1)].shape[0] >= 4 * 10 * 12 + 1 * (24 + 24 + 40)


def test_the_plain_pieces_on_cases_made_by_hand():
    x = torch.tensor([[1.0, 2.0], [3.0, 5.0], [7.0, 11.0]], dtype=torch.float64)
    w = torch.tensor([[10.0, 1.0], [0.0, 2.0]], dtype=torch.float64)  # taps 2: the last column is the current token's
    assert torch.equal(plain.causal_conv(x, w), torch.tensor([[1.0, 4.0], [13.0, 10.0], [37.0, 22.0]], dtype=torch.float64))
    q = torch.tensor([[[1.0, 0.0, 5.0]]], dtype=torch.float64)  # one token at position 1: entries 0 and 1 turn by 1 radian, entry 2 stays
    turned = plain.turn_halves(q, torch.tensor([1]), 2, 10000.0)
    assert torch.allclose(turned, torch.tensor([[[0.5403023058681398, 0.8414709848078965, 5.0]]], dtype=torch.float64))
    assert torch.allclose(plain.turn_halves(turned, torch.tensor([1]), 2, 10000.0, sign=-1.0), q)
    # the router: scores 0.5, 0.3, 0.15, 0.05; the correction lifts output 3 above output 1; groups {0,1} {2,3}: with one group kept
    # only the group of the best choice score can be chosen; weights are the plain scores times the scale
    scores = torch.tensor([[0.5, 0.3, 0.15, 0.05]], dtype=torch.float64)
    w = {"router": torch.eye(4, dtype=torch.float64), "correction": torch.tensor([0.0, 0.0, 0.0, 0.3], dtype=torch.float64)}
    chosen, weight = plain.route(scores.log(), w, "", {"top": 2, "scale": 2.0})
    assert chosen.tolist() == [[0, 3]] and torch.allclose(weight, torch.tensor([[1.0, 0.1]], dtype=torch.float64))
    chosen, weight = plain.route(scores.log(), w, "", {"top": 2, "scale": 2.0, "groups": {"count": 2, "keep": 1}})
    assert chosen.tolist() == [[0, 1]] and torch.allclose(weight, torch.tensor([[1.0, 0.6]], dtype=torch.float64))
    w["correction"] = torch.tensor([-0.6, -0.6, 0.0, 0.0], dtype=torch.float64)  # negative choice scores: an excluded group is not chosen for being "zero"
    chosen, _ = plain.route(scores.log(), w, "", {"top": 2, "scale": 1.0, "groups": {"count": 2, "keep": 1}})
    assert sorted(chosen.tolist()[0]) == [2, 3]
