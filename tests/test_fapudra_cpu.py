"""No device needed: the Fapudra reader in the model registry (a checkpoint directory opens on the host), refused
configurations, and the oracle's own rules on hand-worked cases."""
import numpy as np
import pytest

import fapudra_oracle as O
from yalm_b200 import api


def two_layers():
    return O.make_config(width=40, vocab=50, max_positions=128, layers=[
        O.parallel_layer(mlp=O.moe(ff=12, experts=6, top=2, groups=3, keep=2)),
        O.mamba2_layer(mlp=None)])


def test_directory_checkpoint_opens_through_the_registry(tmp_path):
    cfg = two_layers()
    folder = O.write_checkpoint(str(tmp_path / "m"), cfg, O.random_weights(cfg, 1))
    m = api.Model(folder, 0, api.F32)
    assert m.is_stack() and (m.dim, m.vocab_size, m.n_layers, m.max_seq_len) == (40, 50, 2, 128)
    assert (m.n_experts, m.n_experts_active, m.hidden_dim, m.weight_dtype) == (6, 2, 12, api.F32)
    assert m.n_heads * m.head_dim >= 80          # scratch covers the widest mixer (4 x 20 delta-rule values)
    m.close()
    m = api.Model(folder, 4096)                    # learned positions bound the context
    assert m.weight_dtype == api.BF16 and m.max_seq_len == 128
    m.close()


@pytest.mark.parametrize("edit,what", [
    (lambda c: c["layers"][0].update(type="attention"), "a layer type of another design"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), "heads not a multiple of kv heads"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(vdim=8), "values are keys: one size"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(conv=0), "no convolution taps"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "more selected than the kept groups hold"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4), "experts not a multiple of groups"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "unknown feed-forward kind"),
    (lambda c: c["layers"][1]["mixer"].update(groups=3), "heads not a multiple of groups"),
    (lambda c: c["layers"][1]["mixer"].update(norm_groups=5), "inner size not a multiple of the norm parts"),
])
def test_bad_configurations_are_refused(tmp_path, edit, what):
    cfg = two_layers()
    W = O.random_weights(cfg, 2)
    edit(cfg)
    folder = O.write_checkpoint(str(tmp_path / "m"), cfg, W)
    with pytest.raises(api.YalmError) as e:
        api.Model(folder)
    assert e.value.code == -3, what


def test_distance_buckets_on_worked_cases():
    # 8 rows, far 32: distances 0..3 exact; then 4 rows spread logarithmically over 4..32: boundaries at 4 * 8^(k/4)
    b = [O.distance_bucket(n, 8, 32) for n in range(40)]
    assert b[:4] == [0, 1, 2, 3] and b[4] == 4
    assert b[6] == 4 and b[7] == 5          # 4 * 8^(1/4) = 6.73
    assert b[11] == 5 and b[12] == 6        # 4 * 8^(2/4) = 11.3
    assert b[19] == 6 and b[20] == 7        # 4 * 8^(3/4) = 19.03
    assert b[31] == 7 and b[32] == 7 and b[39] == 7
    assert sorted(set(b)) == list(range(8)) and all(x <= y for x, y in zip(b, b[1:]))


def test_visibility_on_worked_cases():
    assert [j for j in range(10) if O.sees(9, j, 3, 2)] == [0, 1, 7, 8, 9]
    assert [j for j in range(10) if O.sees(2, j, 3, 2)] == [0, 1, 2]
    assert [j for j in range(10) if O.sees(4, j, 3, 0)] == [2, 3, 4]
    assert not O.sees(3, 4, 3, 5)           # never the future, kept or not


def test_group_rule_changes_the_choice():
    z = np.array([5.0, 0.0, 4.0, 3.9, 1.0, 4.5])      # groups of two: their best members 5, 4, 4.5
    ids, w = O.route(z, 2, 3, 2)
    assert sorted(ids) == [0, 5]
    ids, w = O.route(z, 3, 3, 2)
    assert sorted(ids) == [0, 4, 5]                    # expert 2 (4.0) loses to expert 4 (1.0): its group is out
    assert abs(w.sum() - 1) < 1e-12
    ids, w = O.route(z, 3, 3, 3)
    assert sorted(ids) == [0, 2, 5]


def test_convolution_and_shift_start_from_zero():
    x = np.arange(12.0).reshape(4, 3)
    w = np.array([[1.0, 10.0, 100.0]] * 3)
    out = O.causal_conv(x, w)
    assert out[0].tolist() == (100 * x[0]).tolist() and out[2].tolist() == (x[0] + 10 * x[1] + 100 * x[2]).tolist()
    assert O.token_shift(x, np.ones(3))[0].tolist() == [0, 0, 0] and O.token_shift(x, np.ones(3))[2].tolist() == x[1].tolist()
