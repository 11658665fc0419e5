"""Sharded ranking ("predict") and the host-side Engine wrapper, on the GPU.

Scores are checked against the float64 oracle (1e-5 relative) and against predictions recorded
from the reference's torch model; candidate rows must be identical wherever the oracle's scores
are not tied within rounding.  Ties are broken by ascending row, a rule of this engine (the
reference leaves the order undefined)."""

import numpy as np
import pytest

from distributed_kge_poplar_b200 import capi, poplar_kge as kge
from helpers import engine_settings, make_oracle, random_state, write_state
from oracle.step_oracle import StepConfig
from test_engine_gpu import _golden

pytestmark = pytest.mark.gpu
RW = 64


def _predict(engine, cfg, queries, counts, hr, n_best):
    """Host side of predict as the reference's wrapper does it (src/python/poplar_kge.py:782-861):
    queries bucketed by head shard into chunks of hr, per-shard results merged with top-k + sort."""
    n = cfg.n_shard
    out_idx = np.zeros((len(queries), n_best, 2), np.uint32)
    out_score = np.zeros((len(queries), n_best), np.float32)
    per_shard = [np.flatnonzero(queries[:, 0] == s) for s in range(n)]
    for lo in range(0, max(len(x) for x in per_shard), hr):
        head = np.zeros((n, hr), np.uint32)
        rel = np.zeros((n, hr), np.uint32)
        picks = [x[lo : lo + hr] for x in per_shard]
        for s, rows in enumerate(picks):
            head[s, : len(rows)] = queries[rows, 1]
            rel[s, : len(rows)] = queries[rows, 2]
        scores = np.full((n, n, hr, n_best), np.nan, np.float32)
        indices = np.zeros((n, n, hr, n_best), np.uint32)
        engine.run("predict", dict(predict_head=head, predict_relation=rel,
                                   predict_entity_count=np.ascontiguousarray(counts, dtype=np.uint32),
                                   predict_scores=scores, predict_indices=indices))
        for s, rows in enumerate(picks):
            for k, qi in enumerate(rows):
                cand_score = scores[s, :, k].reshape(-1)
                cand_shard = np.repeat(np.arange(n), n_best)
                cand_row = indices[s, :, k].reshape(-1)
                order = np.lexsort((cand_row, cand_shard, -cand_score))[:n_best]
                out_score[qi] = cand_score[order]
                out_idx[qi, :, 0], out_idx[qi, :, 1] = cand_shard[order], cand_row[order]
    return out_idx, out_score


def _clear(score, tol=1e-5):
    """Positions whose score differs from both neighbours by more than rounding."""
    gaps = np.abs(np.diff(score, axis=1)) > tol * np.maximum(1.0, np.abs(score[:, 1:]))
    return np.concatenate([gaps[:, :1], gaps[:, :-1] & gaps[:, 1:], gaps[:, -1:]], axis=1)


@pytest.mark.parametrize("mlp", [0, 21], ids=["plain", "mlp"])
@pytest.mark.parametrize("score_fn,distance_fn", [("TransE", "L1"), ("TransE", "L2"), ("DistMult", "MatMul"), ("ComplEx", "MatMul"), ("RotatE", "L2"),
                                                  ("TransH", "L1")])
def test_predict_matches_oracle(score_fn, distance_fn, mlp):
    if mlp and (score_fn, distance_fn) not in (("TransE", "L2"), ("TransH", "L1")):
        pytest.skip("the feature MLP is covered with two of the score functions")
    cfg = StepConfig(n_shard=3, n_entity=700, n_relation_type=6, embedding_size=36, entity_feature_size=12,
                     batch_size=6, a2a_size=4, score_fn=score_fn, distance_fn=distance_fn, gamma=5.0, feature_mlp_size=mlp,
                     share_feature_networks=not mlp)
    hr, n_best = 8, 5
    state = random_state(cfg, 21, warm=False)
    engine = capi.CEngine(engine_settings(cfg, rw_batch=RW))
    write_state(engine, cfg, state, RW)
    oracle = make_oracle(cfg, state)
    counts = np.array([699, 650, 3])  # a shard with fewer real rows than n_best
    rng = np.random.RandomState(4)
    queries = np.stack([rng.randint(3, size=21), 1 + rng.randint(600, size=21), rng.randint(6, size=21)], axis=1)
    queries[queries[:, 0] == 2, 1] = 1 + queries[queries[:, 0] == 2, 1] % 3
    got_idx, got_score = _predict(engine, cfg, queries, counts, hr, n_best)
    want_idx, want_score = oracle.predict(queries, counts, n_best)
    np.testing.assert_allclose(got_score, want_score, rtol=1e-5, atol=1e-5)
    clear = _clear(want_score)
    np.testing.assert_array_equal(got_idx[clear], want_idx[clear])
    assert np.all(got_idx[..., 1] >= 1) and np.all(got_idx[..., 1] <= counts[got_idx[..., 0]])
    engine.close()


@pytest.mark.parametrize("score_fn,distance_fn", [("TransE", "L2"), ("DistMult", "MatMul")])
@pytest.mark.parametrize("filter_in_scores", ["1", "0"])
def test_predict_in_many_passes_matches_oracle(monkeypatch, score_fn, distance_fn, filter_in_scores):
    """Seven passes of 100 rows over each shard: from the second pass on the queries have
    cut-offs, and a pass's scores reach the lists only through the filter (inside the L2 score
    kernel, or the kernel of its own) and the merge.  n_best = 60 of 100 rows per pass keeps both
    ends busy: passes that overflow nothing and passes whose candidates all pass."""
    monkeypatch.setenv("KGE_PREDICT_PASS_ROWS", "100")
    monkeypatch.setenv("KGE_PREDICT_FILTER_IN_SCORES", filter_in_scores)
    cfg = StepConfig(n_shard=2, n_entity=700, n_relation_type=6, embedding_size=36, entity_feature_size=12,
                     batch_size=6, a2a_size=4, score_fn=score_fn, distance_fn=distance_fn, gamma=5.0)
    hr, n_best = 8, 60
    state = random_state(cfg, 22, warm=False)
    engine = capi.CEngine(engine_settings(cfg, rw_batch=RW, **{"execution.predict_hr_batch_size": hr, "execution.predict_n_best": n_best}))
    write_state(engine, cfg, state, RW)
    oracle = make_oracle(cfg, state)
    counts = np.array([699, 655])
    rng = np.random.RandomState(5)
    queries = np.stack([rng.randint(2, size=13), 1 + rng.randint(600, size=13), rng.randint(6, size=13)], axis=1)
    got_idx, got_score = _predict(engine, cfg, queries, counts, hr, n_best)
    want_idx, want_score = oracle.predict(queries, counts, n_best)
    np.testing.assert_allclose(got_score, want_score, rtol=1e-5, atol=1e-5)
    clear = _clear(want_score)
    np.testing.assert_array_equal(got_idx[clear], want_idx[clear])
    engine.close()


def test_predict_ties_are_broken_by_row():
    cfg = StepConfig(n_shard=1, n_entity=300, n_relation_type=2, embedding_size=8, entity_feature_size=0,
                     batch_size=4, a2a_size=4, score_fn="TransE", distance_fn="L1", gamma=1.0)
    state = random_state(cfg, 3)
    state["entity_data"][0, 1:, :8] = state["entity_data"][0, 1:2, :8]  # every row identical: all scores tie
    engine = capi.CEngine(engine_settings(cfg, rw_batch=RW))
    write_state(engine, cfg, state, RW)
    idx, score = _predict(engine, cfg, np.array([[0, 5, 1]]), np.array([299]), 8, 5)
    np.testing.assert_array_equal(idx[0, :, 1], [1, 2, 3, 4, 5])
    assert np.all(score[0] == score[0, 0])
    engine.close()


@pytest.mark.parametrize("filter_in_scores", ["1", "0"])
def test_predict_ties_across_table_passes_and_shards(monkeypatch, filter_in_scores):
    """Ties between rows that different passes over the table score (a pass is set to 4096 rows, so
    rows 4096 and 4097 meet only in the running top-k, after a cut-off exists) and between rows of
    different shards: the best candidates are returned in ascending (shard, row) order.  Every tied
    row equals the predicted tail exactly, so its distance is an exact zero on any arithmetic.
    Both ways of filtering a pass's scores against the cut-offs: inside the score kernel, and by
    the kernel of its own."""
    monkeypatch.setenv("KGE_PREDICT_PASS_ROWS", "4096")
    monkeypatch.setenv("KGE_PREDICT_FILTER_IN_SCORES", filter_in_scores)
    cfg = StepConfig(n_shard=2, n_entity=4300, n_relation_type=2, embedding_size=8, entity_feature_size=0,
                     batch_size=4, a2a_size=4, score_fn="TransE", distance_fn="L2", gamma=3.0)
    state = random_state(cfg, 8)
    state["relation_embedding"][1] = 0.0          # relation 1: predicted tail = the head row itself
    tied = {0: [4094, 4095, 4096, 4097, 4098, 4200], 1: [2, 4096, 4097]}
    head_row = 7
    for shard, rows in tied.items():
        state["entity_data"][shard, rows, :8] = state["entity_data"][0, head_row, :8]
    engine = capi.CEngine(engine_settings(cfg, rw_batch=RW))
    write_state(engine, cfg, state, RW)
    n_best = 5
    idx, score = _predict(engine, cfg, np.array([[0, head_row, 1]]), np.array([4299, 4299]), 8, n_best)
    np.testing.assert_array_equal(score[0], np.full(n_best, 3.0, np.float32))   # gamma - 0
    np.testing.assert_array_equal(idx[0, :, 0], [0, 0, 0, 0, 0])
    np.testing.assert_array_equal(idx[0, :, 1], [7, 4094, 4095, 4096, 4097])
    # per-shard lists before the merge: shard 1's candidates across its own pass boundary
    scores = np.zeros((2, 2, 8, 5), np.float32)
    indices = np.zeros((2, 2, 8, 5), np.uint32)
    head = np.zeros((2, 8), np.uint32)
    head[0, 0] = head_row
    rel = np.ones((2, 8), np.uint32)
    engine.run("predict", dict(predict_head=head, predict_relation=rel, predict_entity_count=np.array([4299, 4299], np.uint32),
                               predict_scores=scores, predict_indices=indices))
    np.testing.assert_array_equal(indices[0, 1, 0, :3], [2, 4096, 4097])
    np.testing.assert_array_equal(scores[0, 1, 0, :3], [3.0, 3.0, 3.0])
    assert np.all(scores[0, 1, 0, 3:] < 3.0)
    engine.close()


@pytest.mark.parametrize("case", ["demo", "mid"])
def test_predict_matches_reference_model(case):
    g, s, cfg = _golden(case)
    hr, n_best = int(s["execution.predict_hr_batch_size"]), int(s["execution.predict_n_best"])
    engine = capi.CEngine(engine_settings(cfg, rw_batch=RW, **{"execution.predict_hr_batch_size": hr,
                                                              "execution.predict_n_best": n_best}))
    write_state(engine, cfg, {k[len("final/") :]: g[k] for k in g.files if k.startswith("final/")} | {"step": np.zeros(cfg.n_shard, np.uint32)}, RW)
    idx, score = _predict(engine, cfg, g["predict/queries"].astype(np.int64), g["shard_to_count"], hr, n_best)
    np.testing.assert_allclose(score, g["predict/score"], rtol=1e-4, atol=1e-5)
    clear = _clear(g["predict/score"], 1e-4)
    np.testing.assert_array_equal(idx[clear], g["predict/shard_idx"][clear])
    engine.close()


def test_engine_wrapper_operations():
    """The reference's test_engine_ops (tests/python/test_poplar_kge.py:111-172) on the host-side
    twin of its Engine class: initialise, train twice on one batch, variable round trip, features
    read back from the rows, predictions well-formed and sorted."""
    settings = kge.Settings.create_demo()
    settings.seed = 100
    settings.training.learning_rate = 0.01
    settings.prepare()
    m, e = settings.model, settings.execution
    engine = kge.Engine(settings, np.full(m.n_shard, m.n_entity - 1))
    features = engine.random_normal((m.n_shard, m.n_entity, m.entity_feature_size), np.float16)
    features[:, 0, :] = 0
    with pytest.raises(ValueError, match="uninitialised"):
        engine.train_step_loop(None)
    engine.initialise_all(features.astype(np.float32))

    n_step, bshape = e.train_steps_per_program_run, (m.n_shard, e.train_steps_per_program_run)
    remote = np.stack([np.sort(engine.random.permutation(np.arange(1, m.n_entity))[: settings.n_remote])
                       for _ in range(m.n_shard * n_step)]).reshape(bshape + (settings.n_remote,)).astype(np.uint32)
    batch = kge.Batch(remote=remote, a2a=engine.random_integers(settings.n_remote, bshape + (m.n_shard, settings.data.a2a_size)),
                      head=engine.random_integers(settings.n_remote, bshape + (settings.data.batch_size,)),
                      relation=engine.random_integers(m.n_relation_type, bshape + (settings.data.batch_size,)),
                      tail=engine.random_integers(settings.n_tail, bshape + (settings.data.batch_size,)))
    loss_0, _ = engine.train_step_loop(batch)
    loss_1, _ = engine.train_step_loop(batch)
    assert loss_1 < loss_0
    assert engine.read_variable("step")[0] == 2 * n_step

    new_relations = engine.random_normal(engine.variable_to_shape["relation_embedding"])
    assert not np.allclose(engine.read_variable("relation_embedding"), new_relations)
    engine.write_variable("relation_embedding", new_relations)
    np.testing.assert_allclose(engine.read_variable("relation_embedding"), new_relations)
    np.testing.assert_allclose(engine.read_entity_all()[:, :, -m.entity_feature_size :], features.astype(np.float32))

    n_predict = e.predict_hr_batch_size + 5
    queries = np.stack([engine.random_integers(m.n_shard, (n_predict,)), 1 + engine.random_integers(m.n_entity - 1, (n_predict,)),
                        engine.random_integers(m.n_relation_type, (n_predict,))], axis=-1)
    predictions = engine.predict(queries)
    assert predictions.shard_idx.shape == (n_predict, e.predict_n_best, 2)
    assert np.all(np.isin(predictions.shard_idx[:, :, 0], np.arange(m.n_shard)))
    assert np.all(np.isin(predictions.shard_idx[:, :, 1], np.arange(1, m.n_entity)))
    assert predictions.score.shape == (n_predict, e.predict_n_best) and not np.any(np.isnan(predictions.score))
    np.testing.assert_equal(predictions.score, np.sort(predictions.score, axis=-1)[..., ::-1])


def _demo_engine_and_batch(seed):
    settings = kge.Settings.create_demo()
    settings.seed = seed
    settings.training.learning_rate = 0.01
    settings.prepare()
    m, e = settings.model, settings.execution
    engine = kge.Engine(settings, np.full(m.n_shard, m.n_entity - 1))
    bshape = (m.n_shard, e.train_steps_per_program_run)
    draw = np.random.RandomState(seed)
    remote = np.stack([np.sort(draw.permutation(np.arange(1, m.n_entity))[: settings.n_remote])
                       for _ in range(m.n_shard * bshape[1])]).reshape(bshape + (settings.n_remote,)).astype(np.uint32)
    batch = kge.Batch(remote=remote,
                      a2a=draw.randint(settings.n_remote, size=bshape + (m.n_shard, settings.data.a2a_size)).astype(np.uint32),
                      head=draw.randint(settings.n_remote, size=bshape + (settings.data.batch_size,)).astype(np.uint32),
                      relation=draw.randint(m.n_relation_type, size=bshape + (settings.data.batch_size,)).astype(np.uint32),
                      tail=draw.randint(settings.n_tail, size=bshape + (settings.data.batch_size,)).astype(np.uint32))
    return settings, engine, batch


def test_sharded_checkpoint_resumes_bit_exactly(tmp_path):
    """Train, dump one file per shard, train on; a fresh engine restored from the dump and trained
    on the same batches ends in the same state bit for bit (rows with optimiser state, dense
    variables with theirs, step counter, learning-rate schedule)."""
    settings, engine, batch = _demo_engine_and_batch(7)
    m = settings.model
    features = engine.random_normal((m.n_shard, m.n_entity, m.entity_feature_size), np.float16)
    engine.initialise_all(features.astype(np.float32))
    engine.train_step_loop(batch)
    engine.DUMP_CHUNK_BYTES = 37 * 1024  # several ragged chunks per shard
    engine.dump(tmp_path)
    assert sorted(p.name for p in tmp_path.iterdir()) == (
        [f"entity_shard{s:03d}.npy" for s in range(m.n_shard)] + ["manifest.json", "variables.npz"])
    loss_a, lr_a = engine.train_step_loop(batch)
    expected = engine.read_all()

    _, resumed, _ = _demo_engine_and_batch(7)
    with pytest.raises(ValueError, match="uninitialised"):
        resumed.train_step_loop(batch)
    resumed.DUMP_CHUNK_BYTES = 53 * 1024
    resumed.restore(tmp_path)
    loss_b, lr_b = resumed.train_step_loop(batch)
    assert (loss_a, lr_a, engine.step) == (loss_b, lr_b, resumed.step)
    actual = resumed.read_all()
    assert sorted(actual) == sorted(expected)
    for name in expected:
        np.testing.assert_array_equal(actual[name], expected[name], err_msg=name)

    other = kge.Settings.create_demo()
    other.model.embedding_size *= 2
    other.prepare()
    mismatch = kge.Engine(other, np.full(other.model.n_shard, other.model.n_entity - 1))
    with pytest.raises(ValueError, match="row_bytes|embedding_size"):
        mismatch.restore(tmp_path)
    with pytest.raises(ValueError, match="shard_range"):
        engine.engine.run("dump_entity_rows", dict(shard_range=np.array([0, m.n_entity - 1, 2], np.uint32),
                                                   rows=np.zeros((2, engine._entity_layout()[0] // 4), np.uint32)))
