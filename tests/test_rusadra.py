"""The Rusadra design without a GPU: its configuration's keys and refusals, the model it is turned into (run order,
shared pages, tensor names), random model folders, and the plain implementation's own properties (a sequence cut in
two gives the same as in one piece; what lies outside a window has no influence)."""
import copy
import json
import os

import numpy as np
import pytest
import torch

import plain_rusadra as P
from rusadra_configs import RUSADRA, RUSADRA_A, RUSADRA_B, write_rusadra_model

from llm_rs_b200.config import ConfigError, RusadraConfig, load_config, resolve_architecture
from llm_rs_b200.parts import DecoderModel


def test_config_reads_every_key_and_writes_them_back():
    cfg = RusadraConfig.from_dict(RUSADRA_A)
    assert (cfg.vocab, cfg.width, cfg.norm_eps, cfg.logit_softcap) == (211, 64, 1e-5, 12.0)
    assert [l.type for l in cfg.layers] == ["general_delta", "latent_attention", "general_delta", "latent_attention"]
    m = cfg.layers[3].mixer
    assert (m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank, m.window, m.kv_from) == (3, 16, 8, 24, 40, 33, 1)
    assert cfg.layers[2].mlp is None and cfg.layers[3].mlp.top == 3 and cfg.layers[0].mlp.limit == 0.7
    again = RusadraConfig.from_dict(json.loads(json.dumps(cfg.to_dict())))
    assert again == cfg
    assert resolve_architecture(cfg.to_dict()).name == "Rusadra"
    assert "logit_softcap" not in RusadraConfig.from_dict(RUSADRA_B).to_dict()


@pytest.mark.parametrize("change,message", [
    (lambda c: c.pop("vocab"), "vocab missing"),
    (lambda c: c["layers"][0].update(type="conv"), "type must be one of"),
    (lambda c: c["layers"][1]["mixer"].pop("kv_rank"), "kv_rank missing"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=2), "kv_from 2 must name an earlier latent_attention"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "kv_from 3 must name an earlier"),
    (lambda c: c["layers"][3]["mixer"].update(kv_rank=48), "must equal those of layer 1"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "rot.dims 7 must be even"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "router.top 5 exceeds"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "mlp.kind must be 'moe'"),
    (lambda c: c["layers"][0]["mixer"].pop("decay_rank"), "decay projection's rank"),
    (lambda c: c["layers"][0]["mixer"].update(heads=2.5), "heads must be an integer"),
])
def test_config_refusals(change, message):
    raw = copy.deepcopy(RUSADRA_A)
    change(raw)
    with pytest.raises(ConfigError, match=message):
        RusadraConfig.from_dict(raw)


def test_sizes_left_to_the_tensors_are_read_from_their_shapes(tmp_path):
    """config.json without the decay projection's rank: the folder's tensor shapes give it."""
    path = write_rusadra_model("A", str(tmp_path))
    with open(os.path.join(path, "config.json")) as f:
        raw = json.load(f)
    for layer in raw["layers"]:
        layer["mixer"].pop("decay_rank", None)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(raw, f)
    entry, cfg = load_config(path)
    assert entry.name == "Rusadra" and [l.mixer.decay_rank for l in cfg.layers if l.type == "general_delta"] == [8, 5]


def test_spec_run_order_shared_pages_and_names():
    cfg = RusadraConfig.from_dict(RUSADRA_A)
    spec = resolve_architecture(RUSADRA_A).build_spec(cfg)
    assert [s.cache_of for s in spec.run_order] == [None, None, None, 1]
    # Layer 1's pages are kept for the wider window of the layer that reads them; each keeps its own window.
    assert spec.layers[1].mixer.params["cache_window"] == 33 and spec.layers[1].mixer.params["window"] == 20
    assert spec.layers[3].mixer.params["window"] == 33 and spec.layers[3].mixer.params["shares_cache"]
    model = DecoderModel(spec)
    names = {s.name: tuple(s.shape) for s in model.weight_specs()}
    assert names["embed"] == (211, 64) and names["head"] == (211, 64) and names["final.norm"] == (64,)
    assert names["l1.mix.dkv"] == (48, 64) and names["l1.mix.dkv.norm"] == (40,) and "l3.mix.dkv" not in names
    assert names["l1.mix.q"] == (72, 64) and names["l1.mix.g"] == (3, 64) and names["l3.mix.uv"] == (72, 40)
    assert names["l0.mix.w1"] == (8, 64) and names["l0.mix.w2"] == (32, 8) and names["l0.mix.a.b"] == (32,)
    assert names["l0.mlp.e3.down"] == (64, 40) and names["l0.mlp.table"] == (211, 2) and names["l0.shift"] == (64,)
    assert not any(n.startswith("l2.mlp.") or n == "l2.norm2" for n in names)
    needs = model.cache_needs()
    assert needs[0][0] is None and set(needs[0][1].tensors) == {"delta.state", "shift.previous"}
    assert needs[1][0].window == 33 and needs[1][0].plane_widths == (40, 8) and needs[1][0].n_kv_heads == 1
    assert needs[3][0] is None and set(needs[3][1].tensors) == {"shift.previous"}
    # A narrower reader does not shrink what its source keeps.
    spec_b = resolve_architecture(RUSADRA_B).build_spec(RusadraConfig.from_dict(RUSADRA_B))
    assert spec_b.layers[0].mixer.params["cache_window"] == 1000 and spec_b.layers[1].mixer.params["window"] == 7


def test_owners_of_equal_rows_share_a_page_group():
    from llm_rs_b200.cache import plan_groups
    from rusadra_configs import RUSADRA_F
    spec = resolve_architecture(RUSADRA_F).build_spec(RusadraConfig.from_dict(RUSADRA_F))
    needs = DecoderModel(spec).cache_needs()
    groups, entry_group, entry_index = plan_groups(needs, spec.run_order, 8)
    assert len(groups) == 1 and groups[0].entries == [0, 2]
    assert entry_group == [0, None, 0, 0] and entry_index == [0, None, 1, 1]      # the reader sees the second owner's rows


def test_random_folder_has_valid_tables_and_loads_by_name(tmp_path):
    from llm_rs_b200.weights import load_weights
    path = write_rusadra_model("A", str(tmp_path))
    cfg, w = P.load_model_dir(path)
    table = w["l3.mlp.table"]
    assert table.shape == (211, 3) and int(table.min()) >= 0 and int(table.max()) < 3
    assert all(len(set(row)) == 3 for row in table.tolist())
    entry, typed = load_config(path)
    model = DecoderModel(entry.build_spec(typed))
    tensors = load_weights(path, model.weight_specs(), torch.bfloat16, "cpu")
    assert tensors["l0.norm1"].dtype == torch.float32 and tensors["l0.mlp.table"].dtype == torch.int32
    assert tensors["l1.mix.q"].dtype == torch.bfloat16


def test_plain_delta_rule_continues_from_its_state():
    g = torch.Generator().manual_seed(0)
    D, H, d = 24, 2, 8
    m = {"heads": H, "dim": d}
    w = {f"m.{n}": torch.randn(H * d, D, generator=g, dtype=torch.float64) / 5 for n in "rkvga"}
    w.update({"m.w1": torch.randn(4, D, generator=g, dtype=torch.float64), "m.w2": torch.randn(H * d, 4, generator=g, dtype=torch.float64),
              "m.w0": torch.randn(H * d, generator=g, dtype=torch.float64), "m.a.b": torch.randn(H * d, generator=g, dtype=torch.float64),
              "m.norm": torch.randn(H * d, generator=g, dtype=torch.float64), "m.o": torch.randn(D, H * d, generator=g, dtype=torch.float64)})
    x = torch.randn(30, D, generator=g, dtype=torch.float64)
    whole, S = P.general_delta(x, w, "m.", m, 1e-6)
    a, Sa = P.general_delta(x[:11], w, "m.", m, 1e-6)
    b, Sb = P.general_delta(x[11:], w, "m.", m, 1e-6, state=Sa)
    assert torch.allclose(torch.cat([a, b]), whole, atol=1e-12) and torch.allclose(S, Sb, atol=1e-12)
    # The decay lies in (exp(-exp(-1/2)), 1): nothing is ever amplified.
    decay = torch.exp(-np.exp(-0.5) * torch.sigmoid(torch.tanh(x @ w["m.w1"].T) @ w["m.w2"].T + w["m.w0"]))
    assert float(decay.min()) > np.exp(-np.exp(-0.5)) - 1e-12 and float(decay.max()) < 1.0


def test_plain_window_and_shared_rows(tmp_path):
    """Changing a token that lies outside every window of model B's narrow reader changes nothing downstream of it
    alone: checked on the mixer, whose output at position i depends on rows i-6..i only."""
    path = write_rusadra_model("B", str(tmp_path))
    cfg, w = P.load_model_dir(path)
    m0, m1 = cfg["layers"][0]["mixer"], cfg["layers"][1]["mixer"]
    g = torch.Generator().manual_seed(1)
    x = torch.randn(40, cfg["width"], generator=g, dtype=torch.float64)
    kv = P.latent_kv(x, w, "l0.mix.", m0, 1e-6)
    y, _ = P.latent_attention(x, w, "l1.mix.", m1, 1e-6, kv=kv)
    x2 = x.clone()
    x2[10] += 1.0
    kv2 = P.latent_kv(x2, w, "l0.mix.", m0, 1e-6)
    y2, _ = P.latent_attention(x, w, "l1.mix.", m1, 1e-6, kv=kv2)
    changed = (y - y2).abs().amax(1) > 0
    assert changed[10:17].all() and not changed[:10].any() and not changed[17:].any()


def test_plain_rotation_is_relative():
    """Scores between rotated vectors depend on the distance of their positions only."""
    g = torch.Generator().manual_seed(2)
    q, k = torch.randn(1, 12, generator=g, dtype=torch.float64), torch.randn(1, 12, generator=g, dtype=torch.float64)
    def score(pq, pk):
        return float((P.rotate_half(q, torch.tensor([pq]), 1e4, 8) * P.rotate_half(k, torch.tensor([pk]), 1e4, 8)).sum())
    assert abs(score(5, 2) - score(105, 102)) < 1e-9 and abs(score(5, 2) - score(6, 2)) > 1e-6
    assert torch.equal(P.rotate_half(q, torch.tensor([9]), 1e4, 8)[:, 8:], q[:, 8:])
