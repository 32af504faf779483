"""CPU-side checks of the Munazen integration: config reader and registry, rotary frequency tables against the plain restatement,
the weight file reader, the restatement's own causality, and the scheduler driving a decoder that takes prompts in portions."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import munazen_oracle as O  # noqa: E402
import munazen_testlib as L  # noqa: E402


def test_config_reader_and_layer_runs(tmp_path):
    from simplellminference_b200.config import MunazenConfig, read_model_config
    cfg = L.make_config([L.gla_layer(), L.parallel_layer(), L.parallel_layer(ff=None), L.gla_layer(ff=16)], loop={"start": 1, "stop": 3, "times": 3})
    folder = L.write_model(str(tmp_path / "m"), cfg, {"embed": np.zeros((2, 2), np.float32)})
    c = read_model_config(folder)
    assert isinstance(c, MunazenConfig) and c.layer_runs() == O.layer_runs(cfg) == [0, 1, 2, 1, 2, 1, 2, 3]
    assert c.layers[1].left.kv_heads == 2 and c.layers[1].right.conv == 3 and c.layers[2].ff is None and c.layers[3].ff == 16
    assert c.layers[1].left.rot.scaling is None and c.streams == 3 and c.norm_groups == 2
    no_loop = dict(cfg)
    del no_loop["loop"]
    assert MunazenConfig.from_dict(no_loop).layer_runs() == [0, 1, 2, 3]
    bad = L.make_config([dict(L.gla_layer(), type="conv")])
    with pytest.raises(ValueError, match="unknown mixer type"):
        MunazenConfig.from_dict(bad)
    moe = L.make_config([L.gla_layer(ff=8)])
    moe["layers"][0]["mlp"]["kind"] = "experts"
    with pytest.raises(ValueError, match="not part of this design"):
        MunazenConfig.from_dict(moe)
    with pytest.raises(ValueError, match="loop"):
        MunazenConfig.from_dict(L.make_config([L.gla_layer()], loop={"start": 0, "stop": 2, "times": 2}))


def test_registry_names_unknown_architectures(tmp_path):
    from simplellminference_b200.config import read_model_config
    from simplellminference_b200.models import MODEL_CLASSES
    cfg = L.make_config([L.gla_layer()])
    cfg["architecture"] = "SomethingElse"
    folder = L.write_model(str(tmp_path / "x"), cfg, {"embed": np.zeros((2, 2), np.float32)})
    with pytest.raises(KeyError, match="not registered"):
        read_model_config(folder)
    assert "Munazen" in MODEL_CLASSES


@pytest.mark.parametrize("dims,base,scaling", [(48, 500000.0, {"factor": 8.0, "original": 1024, "fast": 32.0, "slow": 1.0}), (8, 10000.0, None),
                                               (64, 10000.0, {"factor": 40.0, "original": 4096, "fast": 32.0, "slow": 1.0}),
                                               (16, 100.0, {"factor": 2.0, "original": 16, "fast": 4.0, "slow": 2.0})])
def test_scaled_rotary_frequencies(dims, base, scaling):
    from simplellminference_b200.layers import yarn_frequencies
    f, mag = yarn_frequencies(dims, base, scaling)
    f0, mag0 = O.rotary_frequencies(dims, base, scaling)
    np.testing.assert_allclose(np.array(f), f0, rtol=1e-14)
    assert abs(mag - mag0) < 1e-15
    if scaling:   # fast pairs keep their frequency, slow ones are divided by the factor
        plain, _ = O.rotary_frequencies(dims, base, None)
        assert np.all(np.array(f) <= plain * (1 + 1e-12)) and np.all(np.array(f) >= plain / scaling["factor"] * (1 - 1e-12))


def test_weight_file_reader_keeps_the_stored_bits(tmp_path):
    from simplellminference_b200 import weights
    cfg = L.make_config([L.parallel_layer()])
    w = L.random_weights(cfg, seed=3)
    folder = L.write_model(str(tmp_path / "m"), cfg, w)
    raw = weights.read_raw(os.path.join(folder, "model.safetensors"))
    assert set(raw) == set(w)
    for name, (dt, shape, a) in raw.items():
        assert dt == "BF16" and shape == w[name].shape
        np.testing.assert_array_equal((a.astype(np.uint32) << 16).view(np.float32), w[name])


def test_restatement_is_causal_and_loops_share_weights():
    cfg = L.make_config([L.gla_layer(), L.parallel_layer()], loop={"start": 0, "stop": 2, "times": 2})
    w = L.random_weights(cfg, seed=5)
    toks = np.random.default_rng(0).integers(0, cfg["vocab"], size=40).tolist()
    full, layers = O.forward(cfg, w, toks, want_layers=True)
    assert layers.shape[0] == 4
    np.testing.assert_allclose(O.forward(cfg, w, toks[:17]), full[:17], rtol=0, atol=1e-9)
    other = list(toks)
    other[30] = (other[30] + 1) % cfg["vocab"]
    np.testing.assert_allclose(O.forward(cfg, w, other)[:30], full[:30], rtol=0, atol=1e-9)
    assert np.abs(O.forward(cfg, w, other)[30:] - full[30:]).max() > 1e-3


class _PortionDecoder:
    """Host-only stand-in with the interface of seqengine.SequenceDecoder: prompts advance by up to `portion` positions per step."""

    def __init__(self, max_seqs, n_pages, page_len, portion):
        from simplellminference_b200.batch import KvPages
        self.max_seqs, self.n_pages, self.page_len, self.portion = max_seqs, n_pages, page_len, portion
        self.max_len = n_pages * page_len
        self.pages = KvPages(n_pages, page_len, max_seqs, n_pages)
        self.req, self.free = {}, list(range(max_seqs))

    free_pages = property(lambda self: self.pages.free)

    def add(self, prompt):
        slot = self.free.pop(0)
        self.req[slot] = dict(prompt=list(prompt), pos=0, out=[], limit=None)
        return slot

    def set_limit(self, slot, positions):
        self.req[slot]["limit"] = positions

    def position(self, slot):
        return self.req[slot]["pos"]

    def tokens(self, slot):
        r = self.req[slot]
        return np.array(r["prompt"][1:min(r["pos"], len(r["prompt"]))] + r["out"], dtype=np.int32)

    def remove(self, slot):
        self.pages.release(slot)
        del self.req[slot]
        self.free.append(slot)

    def step(self, n):
        for _ in range(n):
            for slot, r in self.req.items():
                if r["limit"] is not None and r["pos"] >= r["limit"]:
                    continue
                left = len(r["prompt"]) - r["pos"]
                adv = min(left, self.portion) if left > 0 else 1
                r["pos"] += adv
                self.pages.reserve(slot, r["pos"])
                if r["pos"] >= len(r["prompt"]):
                    r["out"].append(1000 * slot + len(r["out"]))


def test_scheduler_with_a_decoder_that_takes_prompts_in_portions():
    """A request moved by more than one position per step must not run past its end inside a chunk of steps, and its pages must suffice."""
    pytest.importorskip("torch")
    from simplellminference_b200 import _lib
    if not (os.path.exists(_lib.LIB_PATH) or os.path.exists(_lib.SEQ_LIB_PATH)):
        pytest.skip("library not built")
    from simplellminference_b200.scheduler import ContinuousBatcher
    dec = _PortionDecoder(max_seqs=2, n_pages=6, page_len=8, portion=5)
    cb = ContinuousBatcher(dec, chunk=8)
    lens, new = [13, 1, 8, 20], 3
    ids = [cb.submit(list(range(n)), new) for n in lens]
    out = cb.run()
    assert dec.pages.free == 6 and not dec.req
    for rid, n in zip(ids, lens):
        assert len(out[rid]) == n + new - 1
        assert out[rid][:n - 1].tolist() == list(range(1, n))


def test_partial_library_is_self_contained():
    """The library that carries only the ragged-batch kernels must not need a symbol of the translation units it leaves out."""
    import subprocess
    from simplellminference_b200 import _lib
    if not os.path.exists(_lib.SEQ_LIB_PATH):
        pytest.skip("partial library not built")
    out = subprocess.run(["nm", "-D", "--undefined-only", _lib.SEQ_LIB_PATH], capture_output=True, text=True, check=True).stdout
    missing = [ln.split()[-1] for ln in out.splitlines() if " U " in ln and "sllm" in ln]
    assert not missing, missing
