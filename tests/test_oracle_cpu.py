"""Pins the CPU oracle: against results recorded from the reference's own torch model, against
the reference's operator known-answer vectors, against torch autograd for the hand-derived
backward, and (where a checkout of the reference is present) against the reference's own
distance code compiled from its sources."""

import ctypes
from pathlib import Path

import numpy as np
import pytest

from helpers import BATCH_KEYS, check_batch_decodes_to_training_triples, random_batch, random_state
from oracle import step_oracle as so
from oracle.step_oracle import Oracle, StepConfig

GOLDEN = Path(__file__).parent / "golden"


def _golden(case):
    g = np.load(GOLDEN / f"train_{case}.npz")
    s = {k[len("settings/") :]: g[k][()] for k in g.files if k.startswith("settings/")}
    cfg = StepConfig(n_shard=int(s["model.n_shard"]), n_entity=int(s["model.n_entity"]),
                     n_relation_type=int(s["model.n_relation_type"]), embedding_size=int(s["model.embedding_size"]),
                     entity_feature_size=int(s["model.entity_feature_size"]), batch_size=int(s["data.batch_size"]),
                     a2a_size=int(s["data.a2a_size"]), score_fn=str(s["model.score_fn"]),
                     distance_fn=str(s["model.distance_fn"]), gamma=float(s["model.gamma"]),
                     loss_type=str(s["training.loss.type"]), loss_scale=float(s["training.loss_scale"]))
    return g, s, cfg


@pytest.mark.parametrize("case", ["demo", "mid"])
def test_oracle_reproduces_the_reference_model(case):
    """Same protocol and bounds as tests/python/test_poplar_kge.py:175-259 (loss 1e-4, state 1e-4)."""
    g, s, cfg = _golden(case)
    oracle = Oracle(cfg, np.float64)
    oracle.set_state({k[len("initial/") :]: g[k] for k in g.files if k.startswith("initial/")})
    lr = float(s["training.learning_rate"])
    losses = []
    for i in range(int(g["n_loop"])):
        losses.append(oracle.train_step_loop(lr, {k: g[f"batch{i % 3}/{k}"] for k in BATCH_KEYS}).sum())
    np.testing.assert_allclose(losses, g["loss_mean_per_loop"], rtol=1e-4)
    final = oracle.get_state()
    for key in (k[len("final/") :] for k in g.files if k.startswith("final/")):
        delta = final[key] - g[f"initial/{key}"]
        want = g[f"final/{key}"].astype(np.float64) - g[f"initial/{key}"]
        if key == "entity_data":
            delta, want = delta[:, 1:], want[:, 1:]
        assert np.sqrt(np.sum((delta - want) ** 2) / np.sum(want**2)) <= 1e-4, key


@pytest.mark.parametrize("case", ["demo", "mid"])
def test_oracle_predict_matches_the_reference_model(case):
    g, s, cfg = _golden(case)
    oracle = Oracle(cfg, np.float64)
    oracle.set_state({k[len("final/") :]: g[k] for k in g.files if k.startswith("final/")})
    n_best = int(s["execution.predict_n_best"])
    shard_idx, score = oracle.predict(g["predict/queries"], g["shard_to_count"], n_best)
    np.testing.assert_allclose(score, g["predict/score"], rtol=1e-4, atol=1e-5)
    # candidates agree wherever neighbouring scores are not tied within rounding
    want = g["predict/shard_idx"]
    gaps = np.abs(np.diff(g["predict/score"], axis=1))
    clear = np.concatenate([gaps[:, :1] > 1e-4, (gaps[:, :-1] > 1e-4) & (gaps[:, 1:] > 1e-4), gaps[:, -1:] > 1e-4], axis=1)
    np.testing.assert_array_equal(shard_idx[clear], want[clear])


def test_sampler_fixture_decodes_to_training_triples():
    """The routing contract the engine implements, on batches drawn by the reference's sampler:
    remote -> a2a -> exchange -> tail recovers (h, r, t) triples of the training set
    (tests/python/test_poplar_kge_dataset.py:48-80)."""
    for case in ("demo", "mid"):
        f = np.load(GOLDEN / f"sampler_{case}.npz")
        for b in range(2):
            batch = {k: f[f"batch{b}/{k}"] for k in BATCH_KEYS}
            check_batch_decodes_to_training_triples(batch, int(f["n_shard"]), int(f["batch_size"]), f["train_hrt"],
                                                    f["entity_to_shard"], f["entity_to_idx"])


def test_operator_known_answers():
    """tests/pag/testPag.cpp: l1dist :290-319, l2dist :334-369, multiSlice :602-628,
    logSoftmax :775-794, logSigmoid :817-845, allToAll :881-904; testFructose.cpp:57-67."""
    a = np.arange(10, dtype=np.float64).reshape(2, 5)
    b = np.arange(20, dtype=np.float64).reshape(4, 5)
    ones = np.ones((2, 4))
    np.testing.assert_array_equal(so.l1_distance(a, b), [[0, 25, 50, 75], [25, 0, 25, 50]])
    np.testing.assert_array_equal(so.l1_distance_grad(a, b, ones), [[-3] * 5, [-1] * 5])
    np.testing.assert_array_equal(so.l1_distance_grad(b, a, ones.T), [[-1] * 5, [1] * 5, [2] * 5, [2] * 5])
    dist = so.l2_distance(a, b)
    np.testing.assert_allclose(dist, [[0, 11.1803, 22.3607, 33.5410], [11.1803, 0, 11.1803, 22.3607]], atol=1e-4)
    np.testing.assert_allclose(so.l2_distance_grad(a, b, dist, ones), [[-1.3416] * 5, [-0.4472] * 5], atol=1e-4)
    np.testing.assert_allclose(so.l2_distance_grad(b, a, dist.T, ones.T),
                               [[-0.4472] * 5, [0.4472] * 5, [0.8944] * 5, [0.8944] * 5], atol=1e-4)
    np.testing.assert_allclose(
        so.scatter_add_rows(3, np.array([1, 1, 0, 1]), np.array([[0.1, 1], [0.2, 2], [0.3, 3], [0.4, 4]])),
        [[0.3, 3], [0.7, 7], [0, 0]])
    x = np.array([1.0, 1.0, 2.0])
    norm = np.log(2 * np.exp(1.0) + np.exp(2.0))
    logp = so.log_softmax(x)
    np.testing.assert_allclose(logp, [1 - norm, 1 - norm, 2 - norm])
    np.testing.assert_allclose(so.log_softmax_grad(logp, np.array([10.0, 15.0, 5.0])),
                               [10 - 30 * np.exp(1 - norm), 15 - 30 * np.exp(1 - norm), 5 - 30 * np.exp(2 - norm)])
    xs = np.array([-100, -12, -1, 0, 1, 12, 100], np.float64)
    np.testing.assert_allclose(so.log_sigmoid(xs), -np.log1p(np.exp(-xs)), atol=1e-2)
    np.testing.assert_allclose(so.log_sigmoid_grad(xs, np.full(7, 10.0)), 10 / (1 + np.exp(xs)), atol=1e-2)
    blocks = np.array([[[1011, 1012, 1013], [1021, 1022, 1023]], [[2011, 2012, 2013], [2021, 2022, 2023]]], np.float64)
    np.testing.assert_array_equal(so.all_to_all(blocks).reshape(-1),
                                  [1011, 1012, 1013, 2011, 2012, 2013, 1021, 1022, 1023, 2021, 2022, 2023])
    # lpnorm (src/poplar_kge.cpp:389-391) and the reference's pow backward, which gives 0 where the base is 0
    np.testing.assert_allclose(so.lp_norm(np.array([[3.0, -4.0], [0.0, 0.0]]), 2.0), [5.0, 0.0])
    np.testing.assert_allclose(so.lp_norm_grad(np.array([[3.0, -4.0], [0.0, 0.0]]), 2.0, np.array([10.0, 10.0])), [[6.0, -8.0], [0.0, 0.0]])
    np.testing.assert_allclose(so.lp_norm_grad(np.array([[1.0, -2.0, 0.0]]), 1.0, np.array([2.0])), [[2.0, -2.0, 0.0]])
    # softmax cross-entropy of uniform logits over 4 classes is log 4
    cfg = StepConfig(n_shard=1, n_entity=10, n_relation_type=1, embedding_size=2, entity_feature_size=0,
                     batch_size=1, a2a_size=4, loss_type="softmax")
    loss, _ = so.loss_softmax(cfg, np.zeros((1, 4)), np.array([2]))
    np.testing.assert_allclose(loss, np.log(4.0))


VARIANTS = [
    dict(score_fn="TransE", distance_fn="L1", loss_type="logsigmoid"),
    dict(score_fn="TransE", distance_fn="L2", loss_type="softmax", correction_weight=1.0),
    dict(score_fn="TransE", distance_fn="L2", loss_type="logsigmoid", negative_adversarial_scale=2.0),
    dict(score_fn="DistMult", distance_fn="MatMul", loss_type="logsigmoid"),
    dict(score_fn="ComplEx", distance_fn="MatMul", loss_type="softmax", correction_weight=0.3),
    dict(score_fn="TransE", distance_fn="L1", loss_type="softmax", share_feature_networks=False),
    dict(score_fn="TransE", distance_fn="L2", loss_type="softmax", embedding_regularisation=(3.0, 0.02),
         feature_regularisation=(2.0, 0.03), hidden_regularisation=(1.0, 0.01)),
    dict(score_fn="DistMult", distance_fn="MatMul", loss_type="logsigmoid", share_feature_networks=False,
         embedding_regularisation=(2.0, 0.05), feature_regularisation=(2.5, 0.01), hidden_regularisation=(3.0, 0.02)),
    dict(score_fn="TransE", distance_fn="L2", loss_type="softmax", feature_dropout=0.3, feature_regularisation=(2.0, 0.03)),
    dict(score_fn="TransE", distance_fn="L2", loss_type="softmax", feature_mlp_size=10, hidden_regularisation=(2.0, 0.02)),
    dict(score_fn="DistMult", distance_fn="MatMul", loss_type="logsigmoid", share_feature_networks=False, feature_mlp_size=6,
         feature_dropout=0.3),
    dict(score_fn="TransH", distance_fn="L1", loss_type="logsigmoid"),
    dict(score_fn="TransH", distance_fn="L1", loss_type="softmax", correction_weight=1.0, share_feature_networks=False),
]


@pytest.mark.parametrize("variant", VARIANTS, ids=lambda v: "-".join(str(x) for x in v.values()))
def test_hand_derived_backward_matches_autograd(variant):
    """The oracle's manual gradients against torch autograd of the same forward in float64."""
    import torch

    cfg = StepConfig(n_shard=2, n_entity=60, n_relation_type=4, embedding_size=8, entity_feature_size=6,
                     batch_size=6, a2a_size=5, gamma=3.0, **variant)
    state = random_state(cfg, 5)
    batch = random_batch(cfg, 1, 6)
    oracle = Oracle(cfg, np.float64)
    oracle.set_state(state)
    masks = np.random.RandomState(11).uniform(size=(2, cfg.n_shard, cfg.n_remote, cfg.embedding_size)) >= cfg.feature_dropout
    oracle.dropout_mask = lambda step, part: masks[part]
    losses = oracle.train_step(1e-3, *(batch[k][:, 0] for k in BATCH_KEYS))

    n, d = cfg.n_shard, cfg.embedding_size
    t = lambda a: torch.tensor(np.asarray(a, np.float64))  # noqa: E731
    idx = {k: torch.tensor(batch[k][:, 0].astype(np.int64)) for k in BATCH_KEYS}
    rows = t(state["entity_data"])
    value = torch.stack([rows[s, idx["remote"][s], :d] for s in range(n)]).requires_grad_(True)
    feat = torch.stack([rows[s, idx["remote"][s], 3 * d :] for s in range(n)])
    rel = t(state["relation_embedding"]).requires_grad_(True)
    normal = t(state["relation_normal"]).requires_grad_(True) if cfg.score_fn == "TransH" else None
    w = {name: t(state[name]).requires_grad_(True) for name in cfg.projection_names}
    w_h = w[cfg.projection_names[0]]
    w_t = w[cfg.projection_names[-1]]
    fh_h, fh_t = feat @ w_h, feat @ w_t
    mlp_w = {}
    if cfg.feature_mlp_size > 0:  # src/poplar_kge.cpp:453-458
        prefixes = [""] if cfg.share_feature_networks else ["head_", "tail_"]
        mlp_w = {pre + kind: t(state[pre + kind]).requires_grad_(True) for pre in prefixes for kind in ("mlp_up_projection", "mlp_down_projection")}
        boom = lambda fh0, pre: torch.relu(torch.cat([value, fh0], dim=-1) @ mlp_w[pre + "mlp_up_projection"]) @ mlp_w[pre + "mlp_down_projection"]  # noqa: E731
        fh_h, fh_t = boom(fh_h, prefixes[0]), boom(fh_t, prefixes[-1])
    if cfg.feature_dropout > 0:  # kept with probability 1 - p, scaled by 1 / (1 - p); a mask per call
        scale = 1.0 / (1.0 - float(np.float32(cfg.feature_dropout)))
        fh_h, fh_t = fh_h * t(masks[0]) * scale, fh_t * t(masks[1]) * scale
    hid_h, hid_t = value + fh_h, value + fh_t
    heads = torch.stack([hid_h[s, idx["head"][s]] for s in range(n)])
    send = torch.stack([hid_t[s, idx["a2a"][s]] for s in range(n)])
    tails = send.transpose(0, 1).reshape(n, cfg.n_tail, d)

    def norm_sum(x, power):  # rows' (sum |x|^p)^(1/p), summed; a zero row has zero gradient (the reference's pow rule)
        s_ = (x.abs() ** power).sum(-1)
        return (torch.where(s_ > 0, s_, torch.ones_like(s_)) ** (1.0 / power) * (s_ > 0)).sum()

    def regularisers(s):  # both entityHidden calls add their three terms (src/poplar_kge.cpp:463-465)
        out = 0
        for hid, fh in ((hid_h, fh_h), (hid_t, fh_t)):
            for (power, weight), x in ((cfg.embedding_regularisation, value[s]), (cfg.feature_regularisation, fh[s]),
                                       (cfg.hidden_regularisation, hid[s])):
                if weight > 0:
                    out = out + float(np.float32(weight)) * norm_sum(x, power)
        return out

    total = 0
    for s in range(n):
        r = rel[idx["relation"][s]]
        h = heads[s]
        if cfg.score_fn == "TransE":
            p = h + r
        elif cfg.score_fn == "TransH":  # src/poplar_kge.cpp:539-565
            nv = normal[idx["relation"][s]]
            nv = nv / torch.sqrt((nv * nv).sum(-1, keepdim=True))
            p = h - nv * (nv * h).sum(-1, keepdim=True) + r
        elif cfg.score_fn == "DistMult":
            p = h * r
        else:
            half = d // 2
            p = torch.cat([h[:, :half] * r[:, :half] - h[:, half:] * r[:, half:],
                           h[:, :half] * r[:, half:] + h[:, half:] * r[:, :half]], dim=1)
        if cfg.score_fn == "TransH":
            projected = tails[s][None, :, :] - nv[:, None, :] * (nv @ tails[s].T)[:, :, None]
            dist = (p[:, None, :] - projected).abs().sum(-1)
        elif cfg.distance_fn == "MatMul":
            dist = p @ tails[s].T
        else:
            dist = torch.cdist(p, tails[s], p=1 if cfg.distance_fn == "L1" else 2)
        scores = cfg.gamma - dist if cfg.score_fn in ("TransE", "TransH") else dist
        onehot = torch.nn.functional.one_hot(idx["tail"][s], cfg.n_tail).double()
        if cfg.loss_type == "softmax":
            shift = float(np.float32(cfg.correction_weight) * np.float32(so.softmax_correction(cfg))) if cfg.correction_weight else 0.0
            loss = torch.nn.functional.cross_entropy(scores + shift * (1 - onehot), idx["tail"][s], reduction="sum") / (n * cfg.batch_size)
        else:
            T = cfg.n_tail
            w_pos, w_neg = float(np.float32(0.5 * T)), float(np.float32(0.5 * T) / np.float32(T - 1))
            weight = onehot * (w_pos - w_neg) + w_neg
            if cfg.negative_adversarial_scale:
                soft = torch.softmax(float(np.float32(cfg.negative_adversarial_scale)) * scores.detach() - 10000.0 * onehot, dim=1)
                weight = weight * (onehot + (T - 1) * soft)
            loss = -(weight * torch.nn.functional.logsigmoid((2 * onehot - 1) * scores)).sum() / (n * cfg.batch_size * cfg.a2a_size * n)
        loss = loss + regularisers(s)
        np.testing.assert_allclose(float(loss.detach()), losses[s], rtol=1e-10)
        total = total + loss
    total.backward(torch.tensor(float(cfg.loss_scale), dtype=torch.float64))
    np.testing.assert_allclose(oracle.last["d_value"], value.grad.numpy(), rtol=1e-9, atol=1e-12)
    np.testing.assert_allclose(oracle.last["grads"]["relation_embedding"], rel.grad.numpy(), rtol=1e-9, atol=1e-12)
    for name, tensor in mlp_w.items():
        np.testing.assert_allclose(oracle.last["grads"][name], tensor.grad.numpy(), rtol=1e-9, atol=1e-12)
    if normal is not None:
        np.testing.assert_allclose(oracle.last["grads"]["relation_normal"], normal.grad.numpy(), rtol=1e-9, atol=1e-12)
    for name in cfg.projection_names:
        np.testing.assert_allclose(oracle.last["grads"][name], w[name].grad.numpy(), rtol=1e-9, atol=1e-12)


def test_reference_distance_code_agrees_with_the_oracle():
    """oracle/_ref/libref_distance.so is the reference's own l1dist / l2dist (+ gradients) compiled
    from its codelet sources; it exists only where a checkout of the reference was present at
    build time."""
    lib_path = Path(__file__).resolve().parents[1] / "oracle" / "_ref" / "libref_distance.so"
    if not lib_path.exists():
        pytest.skip("reference distance code was not built (no checkout of the reference)")
    lib = ctypes.CDLL(str(lib_path))
    fp = ctypes.POINTER(ctypes.c_float)
    for fn in (lib.ref_l1dist, lib.ref_l2dist):
        fn.restype = ctypes.c_float
        fn.argtypes = [fp, fp, ctypes.c_size_t]
    lib.ref_l1distgrad.restype = lib.ref_l2distgrad.restype = ctypes.c_float
    lib.ref_l1distgrad.argtypes = [ctypes.c_float, fp, fp, ctypes.c_size_t]
    lib.ref_l2distgrad.argtypes = [ctypes.c_float, fp, fp, fp, ctypes.c_size_t]
    rng = np.random.RandomState(0)
    a = rng.normal(size=(7, 33)).astype(np.float32)
    b = rng.normal(size=(9, 33)).astype(np.float32)
    b[2] = a[3]
    g = rng.normal(size=(7, 9)).astype(np.float32)
    ptr = lambda x: x.ctypes.data_as(fp)  # noqa: E731
    l1 = np.array([[lib.ref_l1dist(ptr(a[i]), ptr(b[j]), 33) for j in range(9)] for i in range(7)])
    l2 = np.array([[lib.ref_l2dist(ptr(a[i]), ptr(b[j]), 33) for j in range(9)] for i in range(7)])
    np.testing.assert_allclose(l1, so.l1_distance(a.astype(np.float64), b.astype(np.float64)), rtol=1e-5)
    np.testing.assert_allclose(l2, so.l2_distance(a.astype(np.float64), b.astype(np.float64)), rtol=1e-5, atol=1e-7)
    assert l2[3, 2] == 0
    # gradient vertices: one output element (i, k) from column k of b, the row of distances and of grads
    bt = np.ascontiguousarray(b.T)
    dist32 = np.ascontiguousarray(l2.astype(np.float32))
    g1 = np.array([[lib.ref_l1distgrad(float(a[i, k]), ptr(bt[k]), ptr(g[i]), 9) for k in range(33)] for i in range(7)])
    g2 = np.array([[lib.ref_l2distgrad(float(a[i, k]), ptr(bt[k]), ptr(dist32[i]), ptr(g[i]), 9) for k in range(33)] for i in range(7)])
    a64, b64, g64 = a.astype(np.float64), b.astype(np.float64), g.astype(np.float64)
    np.testing.assert_allclose(g1, so.l1_distance_grad(a64, b64, g64), rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(g2, so.l2_distance_grad(a64, b64, so.l2_distance(a64, b64), g64), rtol=1e-4, atol=1e-5)


CPP_VARIANTS = [
    dict(score_fn="TransE", distance_fn="L1", loss_type="logsigmoid"),
    dict(score_fn="TransE", distance_fn="L2", loss_type="softmax", correction_weight=1.0),
    dict(score_fn="DistMult", distance_fn="MatMul", loss_type="logsigmoid"),
    dict(score_fn="ComplEx", distance_fn="MatMul", loss_type="softmax", correction_weight=0.5, share_feature_networks=False),
]


@pytest.mark.parametrize("variant", CPP_VARIANTS, ids=lambda v: f"{v['score_fn']}-{v['distance_fn']}-{v['loss_type']}")
def test_compiled_restatement_agrees_with_the_pinned_oracle(variant):
    """oracle/csrc/bess_step.cpp (float32, C++/OpenMP: the timed CPU baseline and the checker of the
    full-size GPU cases) against the float64 numpy oracle that the reference's fixtures pin: two
    steps from a warm state, losses and every state tensor.  Bound 5e-6 of the tensor's rms (the
    two agree to about 1e-6; float32 rounding of one step is 1e-7 per operation)."""
    from helpers import random_batch, random_state
    from oracle.cpp_oracle import LIB_PATH, CppOracle

    if not LIB_PATH.exists():
        pytest.skip("oracle/_build/libbess_oracle.so has not been built (python oracle/build.py)")
    cfg = so.StepConfig(n_shard=3, n_entity=200, n_relation_type=6, embedding_size=16, entity_feature_size=12,
                        batch_size=12, a2a_size=7, gamma=4.0, **variant)
    state = random_state(cfg, 3, warm=True)
    batch = random_batch(cfg, 2, 4, pad=3)
    pinned = so.Oracle(cfg, np.float64)
    pinned.set_state(state)
    compiled = CppOracle(cfg)
    compiled.set_state(state)
    want_loss = pinned.train_step_loop(1e-3, batch)
    got_loss = compiled.train_step_loop(1e-3, batch)
    np.testing.assert_allclose(got_loss, want_loss, rtol=2e-6)
    want, got = pinned.get_state(), compiled.get_state()
    assert set(want) == set(got)
    for name in want:
        if name == "step":
            np.testing.assert_array_equal(got[name], want[name])
            continue
        rms = float(np.sqrt(np.mean(np.asarray(want[name], np.float64) ** 2)))
        worst = float(np.max(np.abs(np.asarray(got[name], np.float64) - want[name])))
        assert worst <= 5e-6 * rms, f"{name}: {worst / rms:.2e} of the tensor's rms"


def test_rotate_follows_the_float16_points_of_the_reference():
    """RotatE in the oracle (src/poplar_kge.cpp:516-530): angles, sine and cosine go through
    float16, so the predicted tail is a rotation by the float16-rounded sine / cosine exactly, and
    the angle's gradient (computed in float16 in the reference) agrees with the analytic float64
    gradient to float16 accuracy."""
    cfg = so.StepConfig(n_shard=1, n_entity=10, n_relation_type=3, embedding_size=8, entity_feature_size=0, batch_size=4,
                        a2a_size=4, score_fn="RotatE", distance_fn="L2")
    rng = np.random.RandomState(0)
    h, theta, dp = rng.normal(size=(5, 8)), rng.uniform(-3, 3, size=(5, 4)), rng.normal(size=(5, 8))
    p = so.predict_tail(cfg, h, theta)
    t16 = theta.astype(np.float16).astype(np.float64)
    s, c = np.sin(t16).astype(np.float16).astype(np.float64), np.cos(t16).astype(np.float16).astype(np.float64)
    np.testing.assert_array_equal(p, np.concatenate([h[:, :4] * c - h[:, 4:] * s, h[:, 4:] * c + h[:, :4] * s], axis=1))
    # a rotation keeps the modulus of every complex pair, up to the float16 rounding of sine and cosine
    np.testing.assert_allclose(p[:, :4] ** 2 + p[:, 4:] ** 2, h[:, :4] ** 2 + h[:, 4:] ** 2, rtol=2e-3)
    dh, dtheta = so.predict_tail_grad(cfg, h, theta, dp)
    np.testing.assert_allclose(dh, np.concatenate([dp[:, :4] * c + dp[:, 4:] * s, -dp[:, :4] * s + dp[:, 4:] * c], axis=1), rtol=1e-12)
    analytic = dp[:, :4] * (-h[:, :4] * np.sin(theta) - h[:, 4:] * np.cos(theta)) + dp[:, 4:] * (-h[:, 4:] * np.sin(theta) + h[:, :4] * np.cos(theta))
    np.testing.assert_allclose(dtheta, analytic, rtol=0, atol=4e-3 * np.abs(analytic).max())
    assert dtheta.shape == theta.shape
