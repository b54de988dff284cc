"""The Pusazen design without a GPU: its configuration's keys and refusals, what is read from the folder's tensors,
the model it is turned into (part kinds, pages and state, tensor names), random model folders, and the plain
implementation's own properties (what lies outside a chunk has no influence; the sink only takes weight away; the
running maximum of the matrix memory starts at 0; a router weighs the chosen experts only)."""
import copy
import json
import os

import numpy as np
import pytest
import torch

import plain_pusazen as P
from pusazen_configs import PUSAZEN, PUSAZEN_A, PUSAZEN_B, PUSAZEN_E, write_pusazen_model

from llm_rs_b200.config import ConfigError, PusazenConfig, load_config, resolve_architecture
from llm_rs_b200.parts import DecoderModel


def test_config_reads_every_key_and_writes_them_back():
    cfg = PusazenConfig.from_dict(PUSAZEN_A)
    assert (cfg.vocab, cfg.width, cfg.norm_eps, cfg.alpha, cfg.logit_scale) == (211, 64, 1e-5, 1.8, 0.7)
    assert [l.type for l in cfg.layers] == ["mlstm", "attention", "lightning", "mlstm"]
    m = cfg.layers[1].mixer
    assert (m.heads, m.kv_heads, m.dim, m.vdim, m.scale, m.softcap, m.chunk, m.rot_base, m.rot_dims) == \
        (4, 2, 16, 32, 0.4, 6.0, 20, 10000.0, 8)
    assert cfg.layers[0].mixer.gate_cap == 8.0 and cfg.layers[2].mixer.decay == (0.5, 0.9, 0.99)
    assert cfg.layers[0].mlp.ff == 80 and cfg.layers[2].mlp is None
    assert (cfg.layers[1].mlp.experts, cfg.layers[1].mlp.top, cfg.layers[1].mlp.shared_ff) == (4, 2, 24)
    assert cfg.layers[3].mlp.shared_ff == 0
    again = PusazenConfig.from_dict(json.loads(json.dumps(cfg.to_dict())))
    assert again == cfg
    assert resolve_architecture(cfg.to_dict()).name == "Pusazen"
    e = PusazenConfig.from_dict(PUSAZEN_E).layers[0].mixer      # no mask, no rotation
    assert (e.chunk, e.rot_dims) == (0, 0) and "mask" not in e.to_dict() and "rot" not in e.to_dict()


@pytest.mark.parametrize("change,message", [
    (lambda c: c.pop("width"), "width missing"),
    (lambda c: c["layers"][0].update(type="conv"), "type must be one of"),
    (lambda c: c["layers"][0]["mixer"].pop("gate_cap"), "gate_cap missing"),
    (lambda c: c["layers"][0]["mixer"].update(gate_cap=0.0), "gate_cap must be positive"),
    (lambda c: c["layers"][2]["mixer"].update(decay=[0.5, 0.9]), "one number per head"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "no multiple of 3 kv_heads"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "rot.dims 7 must be even"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=18), "rot.dims 18 must be even and at most"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale missing"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=5), "router.top 5 exceeds"),
    (lambda c: c["layers"][0]["mlp"].update(kind="conv"), "mlp.kind must be 'dense' or 'moe'"),
    (lambda c: c["layers"][0]["mixer"].update(heads=2.5), "heads must be an integer"),
])
def test_config_refusals(change, message):
    raw = copy.deepcopy(PUSAZEN_A)
    change(raw)
    with pytest.raises(ConfigError, match=message):
        PusazenConfig.from_dict(raw)


def test_the_model_it_is_turned_into():
    cfg = PusazenConfig.from_dict(PUSAZEN_A)
    spec = resolve_architecture(cfg.to_dict()).build_spec(cfg)
    assert [l.mixer.kind for l in spec.layers] == ["mlstm", "scored_attention", "lightning", "mlstm"]
    assert [None if l.feed_forward is None else l.feed_forward.kind for l in spec.layers] == ["dense", "moe", None, "moe"]
    assert all(l.block.kind == "postnorm" and l.block.params["alpha"] == 1.8 for l in spec.layers)
    assert spec.layers[2].feed_forward_norm is None and spec.lm_head.params["scale"] == 0.7
    model = DecoderModel(spec)
    needs = model.cache_needs()
    assert needs[1][0].kind == "window" and needs[1][0].window == 20 and needs[1][0].plane_widths == (16, 32)
    assert needs[1][1] is None and needs[0][0] is None
    assert {k: tuple(v) for k, v in needs[0][1].tensors.items()} == {
        "recurrent.state": (2, 16, 24), "recurrent.normaliser": (2, 16), "recurrent.maximum": (2,)}
    assert dict(needs[2][1].tensors) == {"recurrent.state": (3, 8, 16)}
    names = {s.name: tuple(s.shape) for s in model.weight_specs()}
    for name, shape in {"embed": (211, 64), "head": (211, 64), "final.norm": (64,), "l0.ls1": (64,), "l0.ls2": (64,),
                        "l0.mix.i": (2, 64), "l0.mix.f.b": (2,), "l0.mix.norm": (48,), "l0.mlp.up": (80, 64),
                        "l1.mix.q.norm": (64,), "l1.mix.k.norm": (32,), "l1.mix.sink": (4,), "l1.mix.o": (64, 128),
                        "l1.mlp.router": (4, 64), "l1.mlp.router.b": (4,), "l1.mlp.e3.down": (64, 40),
                        "l1.mlp.shared.sg": (1, 64), "l1.mlp.shared.gate": (24, 64), "l2.mix.g": (48, 64),
                        "l2.norm1": (64,), "l3.mlp.e2.gate": (24, 64)}.items():
        assert names.get(name) == shape, (name, names.get(name))
    assert "l2.norm2" not in names and "l2.ls2" not in names and "l3.mlp.shared.sg" not in names
    # An attention layer without a mask keeps every key: its pages are a group of kind "full".
    cfg_e = PusazenConfig.from_dict(PUSAZEN_E)
    needs_e = DecoderModel(resolve_architecture(cfg_e.to_dict()).build_spec(cfg_e)).cache_needs()
    assert needs_e[0][0].kind == "full" and needs_e[1][0].kind == "window"


def test_what_the_folder_holds_decides_the_optional_tensors(tmp_path):
    """A folder without layer-scale vectors and without sinks, and one whose feed-forward-less layer still has a second
    norm: the configuration follows the tensors."""
    from llm_rs_b200.weights.safetensors_io import save_file
    path = write_pusazen_model("A", str(tmp_path))
    cfg, w = P.load_model_dir(path)
    entry, typed = load_config(path)
    assert all(l.layer_scale for l in typed.layers) and typed.layers[1].mixer.sink and not typed.layers[2].lone_norm
    kept = {k: v.to(torch.bfloat16) for k, v in w.items() if ".ls" not in k and not k.endswith("sink")}
    kept["l2.norm2"] = torch.ones(64, dtype=torch.bfloat16)
    save_file(kept, os.path.join(path, "model.safetensors"))
    entry, typed = load_config(path)
    assert not any(l.layer_scale for l in typed.layers) and not typed.layers[1].mixer.sink and typed.layers[2].lone_norm
    names = {s.name for s in DecoderModel(entry.build_spec(typed)).weight_specs()}
    assert names == set(kept)


def test_random_folders_load_and_differ_by_seed(tmp_path):
    for name in PUSAZEN:
        path = write_pusazen_model(name, str(tmp_path))
        entry, typed = load_config(path)
        assert entry.name == "Pusazen" and typed.to_dict()["layers"] == PUSAZEN[name][0]["layers"]
        cfg, w = P.load_model_dir(path)
        logits = P.forward(cfg, w, list(range(12)))
        assert logits.shape == (12, cfg["vocab"]) and bool(torch.isfinite(logits).all())


# ---- the plain implementation's own properties ----------------------------------------------------------
def _attention_weights(g, D, m):
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    r = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    return {"m.q": r(H * d, D) / D ** 0.5, "m.k": r(G * d, D) / D ** 0.5, "m.v": r(G * dv, D) / D ** 0.5,
            "m.o": r(D, H * dv) / (H * dv) ** 0.5, "m.q.norm": 1 + 0.2 * r(H * d), "m.k.norm": 1 + 0.2 * r(G * d),
            "m.sink": r(H)}


def test_plain_attention_sees_its_own_chunk_only_and_the_sink_only_takes_weight_away():
    g = torch.Generator().manual_seed(0)
    D = 32
    m = {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 12, "scale": 0.5, "softcap": 5.0, "mask": {"size": 6},
         "rot": {"base": 100.0, "dims": 4}}
    w = _attention_weights(g, D, m)
    x = torch.randn(20, D, generator=g, dtype=torch.float64)
    y = P.attention(x, w, "m.", m, 1e-6)
    x2 = x.clone()
    x2[:12] = torch.randn(12, D, generator=g, dtype=torch.float64)      # everything before the chunk 12..17
    y2 = P.attention(x2, w, "m.", m, 1e-6)
    assert torch.equal(y[12:18], y2[12:18]) and not torch.allclose(y[11], y2[11])
    x3 = x.clone()
    x3[11] += 1.0                                                       # the last position of the chunk before
    assert torch.equal(P.attention(x3, w, "m.", m, 1e-6)[12:], y[12:])
    # A sink far below every score changes nothing; one far above leaves nothing.
    low, high = dict(w), dict(w)
    low["m.sink"] = torch.full((4,), -1e4, dtype=torch.float64)
    high["m.sink"] = torch.full((4,), 1e4, dtype=torch.float64)
    w0 = dict(w)
    w0["m.sink"] = torch.full((4,), -1e30, dtype=torch.float64)
    assert torch.allclose(P.attention(x, low, "m.", m, 1e-6), P.attention(x, w0, "m.", m, 1e-6), atol=1e-12)
    assert float(P.attention(x, high, "m.", m, 1e-6).abs().max()) < 1e-100
    # With the sink at the score's level a lone key (first of a chunk) gets about half the weight.
    assert not torch.allclose(y[12], P.attention(x, w0, "m.", m, 1e-6)[12])


def test_plain_rotation_pairs_channel_i_with_i_plus_half_and_leaves_the_rest():
    x = torch.arange(2 * 1 * 8, dtype=torch.float64).view(2, 1, 8) + 1.0
    y = P.rotate_half(x, 4, 100.0)
    assert torch.equal(y[0], x[0]) and torch.equal(y[1, 0, 4:], x[1, 0, 4:])      # position 0; channels beyond dims
    a0, a1 = 1.0, 100.0 ** (-2.0 / 4)
    u, v = x[1, 0, 0], x[1, 0, 2]
    assert abs(float(y[1, 0, 0]) - float(u * np.cos(a0) - v * np.sin(a0))) < 1e-12
    assert abs(float(y[1, 0, 2]) - float(v * np.cos(a0) + u * np.sin(a0))) < 1e-12
    u, v = x[1, 0, 1], x[1, 0, 3]
    assert abs(float(y[1, 0, 1]) - float(u * np.cos(a1) - v * np.sin(a1))) < 1e-12


def test_plain_matrix_memory_starts_its_maximum_at_zero():
    """One token, a strongly negative input gate: with the maximum started at 0 the gain is exp(i) and the
    denominator's floor is 1, so the output before the head's norm is tiny; the norm then shows its eps."""
    g = torch.Generator().manual_seed(1)
    D, m = 16, {"heads": 1, "dim": 4, "vdim": 4, "gate_cap": 20.0}
    r = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    w = {"m.q": r(4, D), "m.k": r(4, D), "m.v": r(4, D), "m.g": r(4, D), "m.o": torch.eye(D, 4, dtype=torch.float64),
         "m.norm": torch.ones(4, dtype=torch.float64), "m.i": torch.zeros(1, D, dtype=torch.float64),
         "m.i.b": torch.tensor([-18.0], dtype=torch.float64), "m.f": torch.zeros(1, D, dtype=torch.float64),
         "m.f.b": torch.tensor([0.0], dtype=torch.float64)}
    x = r(1, D)
    small = P.mlstm(x, w, "m.", m, 1e-6)
    w["m.i.b"] = torch.tensor([0.0], dtype=torch.float64)
    usual = P.mlstm(x, w, "m.", m, 1e-6)
    # exp(-18) * |q . k| * |v| against sqrt(eps): the output shrinks by orders of magnitude instead of keeping its size.
    assert float(small.abs().max()) < 2e-2 * float(usual.abs().max())


def test_plain_router_weighs_the_chosen_only_and_adds_the_gated_shared_expert():
    g = torch.Generator().manual_seed(2)
    D, F = 8, 6
    r = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    w = {"f.router": torch.zeros(3, D, dtype=torch.float64), "f.router.b": torch.tensor([1.0, 3.0, 2.0], dtype=torch.float64)}
    for e in range(3):
        w.update({f"f.e{e}.gate": r(F, D), f"f.e{e}.up": r(F, D), f"f.e{e}.down": r(D, F)})
    x = r(2, D)
    f = {"router": {"experts": 3, "top": 2}}
    p = torch.softmax(torch.tensor([3.0, 2.0], dtype=torch.float64), 0)
    want = p[0] * P.gated_expert(x, w, "f.e1.") + p[1] * P.gated_expert(x, w, "f.e2.")
    assert torch.allclose(P.moe_ff(x, w, "f.", f), want, atol=1e-12)
    w.update({"f.shared.gate": r(4, D), "f.shared.up": r(4, D), "f.shared.down": r(D, 4), "f.shared.sg": r(1, D)})
    f["shared"] = {"ff": 4}
    extra = P.gated_expert(x, w, "f.shared.") * torch.sigmoid(x @ w["f.shared.sg"].T)
    assert torch.allclose(P.moe_ff(x, w, "f.", f), want + extra, atol=1e-12)
