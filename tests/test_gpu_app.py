"""The GPU linear-method application end to end from a text configuration."""
import glob

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

CONF = """
training_data {{ format: TEXT text: SPARSE_BINARY file: "{train}/part.*" }}
model_output {{ format: TEXT file: "{out}/model" }}
loss {{ type: LOGIT }}
penalty {{ type: L1 lambda: 0.5 lambda: 0.01 }}
learning_rate {{ type: DECAY alpha: 0.1 beta: 1 }}
async_sgd {{ algo: FTRL minibatch: 500 num_data_pass: 3 max_delay: 1
  push_filter {{ type: KEY_CACHING }} }}
"""
CONF_DARLIN = """
training_data {{ format: TEXT text: SPARSE_BINARY file: "{train}/part.*" }}
model_output {{ format: TEXT file: "{out}/darlin" }}
penalty {{ type: L1 lambda: 2 }}
learning_rate {{ type: CONSTANT alpha: 0.5 }}
darlin {{ max_pass_of_data: 8 epsilon: 1e-5 max_block_delay: 0 tail_feature_freq: 2 feature_block_ratio: 1
  save_model_every_n_iter: 3 }}
"""
CONF_EVAL = """
validation_data {{ format: TEXT text: SPARSE_BINARY file: "{train}/part.*" }}
model_input {{ format: TEXT file: "{out}/{name}_S.*" }}
"""


def test_async_sgd_darlin_and_evaluation_apps(cuda_lib, tmp_path, monkeypatch):
    from parameter_server_b200.app import linear
    from parameter_server_b200.system import core
    from parameter_server_b200.utils.textdata import write_sparse_binary
    monkeypatch.setenv("PSB_LOG2_TABLE", "14")
    monkeypatch.setenv("PSB_MAX_NNZ_PER_ROW", "16")
    monkeypatch.setenv("PSB_DARLIN_BLOCK", "128")
    write_sparse_binary(str(tmp_path / "train"), 3, 1500, 12, 400, seed=1)
    res = linear.run_async_sgd(core.parse_text_proto(CONF.format(train=tmp_path / "train", out=tmp_path)), verbose=False)
    assert res["examples"] == 3 * 3 * 1500
    lines = open(glob.glob(str(tmp_path / "model_S0"))[0]).read().splitlines()
    assert len(lines) > 10 and all(len(l.split("\t")) == 2 for l in lines)
    ev = linear.run_evaluation(core.parse_text_proto(CONF_EVAL.format(train=tmp_path / "train", out=tmp_path, name="model")), verbose=False)
    assert ev["auc"] > 0.68 and ev["logloss"] < 0.67
    hist = linear.run_darlin(core.parse_text_proto(CONF_DARLIN.format(train=tmp_path / "train", out=tmp_path)), verbose=False)
    assert hist[-1]["objective"] < 0.95 * 4500 * np.log(2)
    assert glob.glob(str(tmp_path / "darlin_iter_2_S0")), "no intermediate model after the third pass"
    ev2 = linear.run_evaluation(core.parse_text_proto(CONF_EVAL.format(train=tmp_path / "train", out=tmp_path, name="darlin")), verbose=False)
    assert ev2["auc"] > 0.68
