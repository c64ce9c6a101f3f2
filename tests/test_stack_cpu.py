"""No device needed: the model registry and the configuration reader of the layered architectures (a checkpoint directory
opens on the host; only cuda() needs a GPU), the oracle's own visibility rule on hand-worked cases, and the checkpoint
writer / bf16 helpers the GPU tests rely on."""
import json
import os

import numpy as np
import pytest

import stack_oracle as O
from yalm_b200 import api


def two_layers():
    return O.make_config(width=64, vocab=50, max_positions=128, layers=[
        O.attn_layer(heads=4, kv_heads=2, dim=8, vdim=12, window=6, pool=2, mlp=O.dense(ff=20)),
        O.attn_layer(heads=2, kv_heads=1, dim=16, vdim=4, window=9, pool=3, v_mix=False, mlp=O.moe(ff=10, experts=6, top=2))])


def test_directory_checkpoint_opens_through_the_registry(tmp_path):
    cfg = two_layers()
    folder = O.write_checkpoint(str(tmp_path / "m"), cfg, O.random_weights(cfg, 1))
    m = api.Model(folder, 0, api.F32)
    assert m.is_stack() and (m.dim, m.vocab_size, m.n_layers, m.max_seq_len) == (64, 50, 2, 128)
    assert (m.n_experts, m.n_experts_active, m.hidden_dim, m.weight_dtype) == (6, 2, 20, api.F32)
    assert m.n_heads * m.head_dim >= 48          # scratch covers the widest layer's q (4 x 8, 2 x 16) and attention output (4 x 12)
    m.close()
    m = api.Model(folder, 40)                      # dtype as stored, context below the model's limit
    assert m.weight_dtype == api.BF16 and m.max_seq_len == 40
    m.close()
    m = api.Model(folder, 4096)                    # learned positions bound the context
    assert m.max_seq_len == 128
    m.close()


@pytest.mark.parametrize("edit,what", [
    (lambda c: c.update(architecture="NoSuchDesign"), "unknown architecture"),
    (lambda c: c["layers"][0].update(type="recurrent"), "unknown layer type"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "heads not a multiple of kv heads"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=7), "more selected than experts"),
    (lambda c: c["layers"][0]["mlp"].update(kind="conv"), "unknown feed-forward kind"),
    (lambda c: c.update(width=0), "no width"),
])
def test_bad_configurations_are_refused(tmp_path, edit, what):
    cfg = two_layers()
    W = O.random_weights(cfg, 2)
    edit(cfg)
    folder = O.write_checkpoint(str(tmp_path / "m"), cfg, W)
    with pytest.raises(api.YalmError) as e:
        api.Model(folder)
    assert e.value.code == -3, what


def test_config_json_escapes_and_unknown_keys(tmp_path):
    cfg = two_layers()
    cfg["note"] = {"text": "a \"quoted\" \\ string é", "list": [1, 2.5e3, True, None, {"deep": []}]}
    folder = O.write_checkpoint(str(tmp_path / "m"), cfg, O.random_weights(cfg, 3))
    m = api.Model(folder)
    assert m.n_layers == 2
    m.close()
    with open(os.path.join(folder, "config.json"), "w") as f:
        f.write(json.dumps(cfg)[:-1])                 # truncated
    with pytest.raises(api.YalmError):
        api.Model(folder)


def test_visibility_rule_on_worked_cases():
    # window 4, blocks of 2: position 7 sees tokens 4..7 and the blocks that end at or before 3: {0,1} and {2,3}
    assert O.visible(7, 4, 2) == ([4, 5, 6, 7], [0, 1])
    # position 6 sees 3..6; token 2 has left the window, but its block {2,3} is not wholly before it: token 2 is not seen at all
    assert O.visible(6, 4, 2) == ([3, 4, 5, 6], [0])
    assert O.visible(3, 4, 2) == ([0, 1, 2, 3], [])
    assert O.visible(5, 4, 2) == ([2, 3, 4, 5], [0])
    assert O.visible(9, 0, 0) == (list(range(10)), [])
    assert O.visible(5, 2, 0) == ([4, 5], [])
    assert O.visible(4, 1, 1) == ([4], [0, 1, 2, 3])           # blocks of one token: everything older is seen through its "mean"
    # with blocks of one token the pooled path is full causal attention
    rng = np.random.default_rng(0)
    q, k, v = rng.standard_normal((9, 2, 4)), rng.standard_normal((9, 1, 4)), rng.standard_normal((9, 1, 3))
    np.testing.assert_allclose(O.window_pool_attention(q, k, v, 3, 1, 0.5), O.window_pool_attention(q, k, v, 0, 0, 0.5), atol=1e-12)


def test_bf16_helpers_round_to_nearest_even():
    a = np.array([1.0, 1.00390625, 1.01171875, -3.0e38, 1e-40, 0.0], np.float32)    # 1 + 2^-8 is a tie: rounds to even (1.0)
    r = O.round_bf16(a)
    assert r[0] == 1.0 and r[1] == 1.0 and r[2] == 1.015625 and r[5] == 0.0
    assert np.all(O.round_bf16(r) == r)
    cfg = two_layers()
    for v in O.random_weights(cfg, 4).values():
        assert np.array_equal(O.round_bf16(v), np.asarray(v, np.float64))
