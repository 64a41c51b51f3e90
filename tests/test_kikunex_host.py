"""Kikunex without a GPU: the float64 restatement's own pieces, the model-folder checks of the loader."""
import math
import subprocess

import numpy as np
import pytest

import kikunex_oracle as ko


@pytest.fixture(scope="module")
def tools():
    from kuiperllama_b200 import build
    return build.build_seq_tools()


def small():
    layers = [(ko.latent_mixer(), ko.moe_mlp()), (ko.lightning_mixer(), ko.dense_mlp())]
    cfg = ko.make_config(layers=layers, loop=(0, 1, 2))
    return cfg, ko.make_weights(cfg)


def test_missing_tensors_and_unknown_mixers_are_reported(tools, tmp_path):
    cfg, w = small()
    for missing in ("l0.mix.dkv.norm", "l0.shift", "l1.mix.norm", "l1.mlp.act", "l0.mlp.e3.down", "embed.norm"):
        d = ko.write_model(tmp_path / missing, cfg, {k: v for k, v in w.items() if k != missing})
        r = subprocess.run([str(tools / "kuiper_trace"), "--model", str(d), "--out", str(tmp_path), "--dtype", "float32"],
                           capture_output=True, text=True)
        assert r.returncode == 2 and missing in r.stderr, (missing, r.stderr)
    bad = dict(cfg, layers=[dict(cfg["layers"][0], type="convolution")])
    d = ko.write_model(tmp_path / "bad", bad, w)
    r = subprocess.run([str(tools / "kuiper_trace"), "--model", str(d), "--out", str(tmp_path), "--dtype", "float32"],
                       capture_output=True, text=True)
    assert r.returncode == 2 and "convolution" in r.stderr


def test_layer_runs():
    cfg = ko.make_config(layers=[(ko.lightning_mixer(), None)] * 4, loop=(1, 3, 3))
    assert ko.layer_runs(cfg) == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (1, 2), (2, None), (3, None)]
    assert ko.layer_runs(ko.make_config(layers=[(ko.lightning_mixer(), None)] * 2)) == [(0, None), (1, None)]


def test_router_groups():
    """Six experts in three groups of two; the best two groups by the sum of their two choice scores are kept."""
    w = {"p.router": np.eye(6), "p.correction": np.array([0.0, 0.0, 0.0, 0.0, 0.3, 0.3])}
    h = np.array([[3.0, 2.0, 2.5, 2.4, 0.5, 0.4]])
    idx, wt = ko.route(h, w, "p.", {"experts": 6, "top": 2, "scale": 2.0, "groups": {"count": 3, "keep": 1}})
    assert list(idx[0]) == [2, 3]  # group 1 has the largest sum although expert 0 has the largest score
    assert np.allclose(wt[0], 2.0 / (1.0 + np.exp(-np.array([2.5, 2.4]))))
    idx, _ = ko.route(h, w, "p.", {"experts": 6, "top": 2, "scale": 2.0})
    assert list(idx[0]) == [0, 2]


def test_oracle_pieces():
    """The restatement's own pieces against closed forms."""
    assert math.isclose(ko.xielu(np.array([2.0]), 0.0, 0.0)[0], math.log(2.0) * 4 + 1.0)
    z = -1.5
    assert math.isclose(ko.xielu(np.array([z]), 0.3, 0.0)[0], (0.5 + math.log(2.0)) * (math.exp(z) - 1 - z) + z / 2)
    v = np.arange(8, dtype=np.float64)[None, :] + 1
    r = ko.rotate(v, np.array([3.0]), 4, 100.0)
    a0, a1 = 3.0, 3.0 * 100.0 ** -0.5
    assert np.allclose(r[0, :4], [1 * math.cos(a0) - 3 * math.sin(a0), 2 * math.cos(a1) - 4 * math.sin(a1),
                                  3 * math.cos(a0) + 1 * math.sin(a0), 4 * math.cos(a1) + 2 * math.sin(a1)])
    assert np.allclose(r[0, 4:], v[0, 4:])
