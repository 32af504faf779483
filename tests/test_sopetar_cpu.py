"""CPU-side checks of the Sopetar integration: config reader and registry, the distance slopes against the plain restatement, and the
restatement's own properties (visibility, causality, the sink's share, independence of hidden positions)."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import sopetar_oracle as O  # noqa: E402
import sopetar_testlib as L  # noqa: E402


def test_config_reader(tmp_path):
    from simplellminference_b200.config import SopetarConfig, read_model_config
    cfg = L.make_config([L.attention_layer(v_mix=True), L.latent_layer(rot_dims=4, keep_first=2, ff=None), L.attention_layer(size=None, softcap=0, v_mix=True)])
    folder = L.write_model(str(tmp_path / "m"), cfg, {"embed": np.zeros((2, 2), np.float32)})
    c = read_model_config(folder)
    assert isinstance(c, SopetarConfig) and c.embedding_scale == 2.5 and c.norm_eps == 1e-5 and len(c.layers) == 3
    a, b, e = (l.mixer for l in c.layers)
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.softcap, a.mask.size, a.mask.keep_first, a.v_mix) == (4, 2, 16, 24, 30.0, 20, 3, True)
    assert (b.heads, b.dim, b.rot_dim, b.vdim, b.kv_rank, b.rot.dims, b.rot.base, b.mask.size, b.mask.keep_first) == (3, 8, 12, 20, 40, 4, 1000.0, 20, 2)
    assert e.mask.size is None and e.mask.keep_first == 0 and e.softcap == 0.0
    assert c.layers[0].mlp.ff == 40 and c.layers[0].mlp.limit == 1.25 and c.layers[1].mlp is None
    with pytest.raises(ValueError, match="unknown mixer type"):
        SopetarConfig.from_dict(L.make_config([dict(L.latent_layer(), type="conv")]))
    moe = L.make_config([L.latent_layer()])
    moe["layers"][0]["mlp"]["kind"] = "experts"
    with pytest.raises(ValueError, match="not part of this design"):
        SopetarConfig.from_dict(moe)
    with pytest.raises(ValueError, match="rotary dimensions"):
        SopetarConfig.from_dict(L.make_config([L.latent_layer(rot_dim=8, rot_dims=10)]))
    with pytest.raises(ValueError, match="do not divide"):
        SopetarConfig.from_dict(L.make_config([L.attention_layer(heads=5, kv_heads=2)]))
    with pytest.raises(ValueError, match="same key/value heads"):
        SopetarConfig.from_dict(L.make_config([L.attention_layer(v_mix=True), L.attention_layer(vdim=8, v_mix=True)]))


def test_registry_knows_the_design():
    from simplellminference_b200.config import CONFIG_READERS
    from simplellminference_b200.models import MODEL_CLASSES
    assert "Sopetar" in MODEL_CLASSES and "Sopetar" in CONFIG_READERS and "Munazen" in MODEL_CLASSES


@pytest.mark.parametrize("heads", [1, 2, 6, 8, 12])
def test_distance_slopes(heads):
    from simplellminference_b200.layers import distance_slopes
    np.testing.assert_allclose(distance_slopes(heads), O.distance_slopes(heads), rtol=1e-15)
    assert abs(distance_slopes(heads)[-1] - 2.0 ** -8) < 1e-18


def test_visibility():
    see = O.visible(12, size=4, keep_first=2)
    for i in range(12):
        for j in range(12):
            assert see[i, j] == (j <= i and (i - j < 4 or j < 2))
    assert O.visible(5).tolist() == np.tril(np.ones((5, 5), bool)).tolist()
    assert O.visible(6, size=1).tolist() == np.eye(6, dtype=bool).tolist()


def test_restatement_is_causal_and_blind_outside_its_windows():
    """Later tokens do not change earlier logits; a token that no window of any layer reaches (directly or through the layers between)
    does not change a late logit, the one just inside does."""
    cfg = L.make_config([L.attention_layer(size=5, keep_first=0, v_mix=True), L.latent_layer(size=4), L.attention_layer(size=3, keep_first=0, v_mix=True)])
    w = {k: v.astype(np.float64) for k, v in L.random_weights(cfg, seed=1).items()}
    rng = np.random.default_rng(2)
    toks = rng.integers(0, cfg["vocab"], size=40).tolist()
    full = O.forward(cfg, w, toks)
    np.testing.assert_allclose(O.forward(cfg, w, toks[:25]), full[:25], rtol=1e-9, atol=1e-9)
    reach = (5 - 1) + (4 - 1) + (3 - 1)                     # the farthest position the last token depends on
    other = list(toks)
    other[39 - reach - 1] = (other[39 - reach - 1] + 1) % cfg["vocab"]
    np.testing.assert_allclose(O.forward(cfg, w, other)[39], full[39], rtol=1e-9, atol=1e-9)
    other = list(toks)
    other[39 - reach] = (other[39 - reach] + 1) % cfg["vocab"]
    assert np.abs(O.forward(cfg, w, other)[39] - full[39]).max() > 1e-9


def test_sink_takes_its_share():
    """With one visible key the softmax weight is 1 / (1 + exp(sink - score)): the first token's output shrinks accordingly."""
    layer = L.latent_layer(heads=1, size=8)
    cfg = L.make_config([layer])
    w = {k: v.astype(np.float64) for k, v in L.random_weights(cfg, seed=4).items()}
    h = np.random.default_rng(5).standard_normal((1, cfg["width"]))
    with_sink = O.latent_attention(h, w, "l0.mix.", layer["mixer"], 1e-5)
    w2 = dict(w)
    w2["l0.mix.sink"] = np.array([-1e9])
    without = O.latent_attention(h, w2, "l0.mix.", layer["mixer"], 1e-5)
    ratio = (with_sink * without).sum() / (without * without).sum()
    assert 0.0 < ratio < 1.0 and np.allclose(with_sink, ratio * without)


def test_depth_average_of_the_restatement():
    """A model whose layers add nothing (zero output projections and down projections) passes on coefficient sums of the embedding output."""
    cfg = L.make_config([L.latent_layer(), L.attention_layer()])
    w = {k: v.astype(np.float64) for k, v in L.random_weights(cfg, seed=6).items()}
    for i in range(2):
        w[f"l{i}.mix.o"] *= 0.0
        w[f"l{i}.mlp.down"] *= 0.0
        w[f"l{i}.mlp.down.b"] *= 0.0
    taps = []
    O.forward(cfg, w, [3, 4], taps)
    x0 = w["embed"][[3, 4]] * cfg["embedding"]["scale"]
    s0 = w["l0.dwa"].sum()
    np.testing.assert_allclose(taps[0], s0 * x0, rtol=1e-12)
    np.testing.assert_allclose(taps[1], (w["l1.dwa"][0] + w["l1.dwa"][1] + w["l1.dwa"][2] * s0) * x0, rtol=1e-12)
