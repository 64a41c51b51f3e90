"""Host side of the batched models without a GPU: the tools build, the model folder readers reject what they must."""
import json
import subprocess

import pytest

from fobolorn_oracle import layer_order, make_config, make_weights, write_model


@pytest.fixture(scope="module")
def tools():
    from kuiperllama_b200 import build
    return build.build_seq_tools()


def test_tools_build_and_refuse_bad_arguments(tools):
    r = subprocess.run([str(tools / "kuiper_trace")], capture_output=True, text=True)
    assert r.returncode == 2 and "usage" in r.stderr
    r = subprocess.run([str(tools / "kuiper_trace"), "--model", "/nonexistent", "--out", "/tmp", "--dtype", "float32"],
                       capture_output=True, text=True)
    assert r.returncode == 2 and "config.json" in r.stderr


def test_unknown_architecture_and_missing_tensor_are_reported(tools, tmp_path):
    cfg = make_config(layers=1)
    w = make_weights(cfg)
    bad = dict(cfg, architecture="SomethingElse")
    d = write_model(tmp_path / "a", bad, w)
    r = subprocess.run([str(tools / "kuiper_trace"), "--model", str(d), "--out", str(tmp_path), "--dtype", "float32"],
                       capture_output=True, text=True)
    assert r.returncode == 2 and "SomethingElse" in r.stderr
    w2 = {k: v for k, v in w.items() if k != "l0.mix.q.norm"}
    d = write_model(tmp_path / "b", cfg, w2)
    r = subprocess.run([str(tools / "kuiper_trace"), "--model", str(d), "--out", str(tmp_path), "--dtype", "float32"],
                       capture_output=True, text=True)
    assert r.returncode == 2 and "l0.mix.q.norm" in r.stderr


def test_oracle_layer_order():
    cfg = make_config(layers=4, loop=(1, 3, 3))
    assert layer_order(cfg) == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (1, 2), (2, None), (3, None)]
    assert layer_order(make_config(layers=2)) == [(0, None), (1, None)]
