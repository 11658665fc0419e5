"""The BESS batch sampler on the device against the invariants of the reference's sampler tests
(tests/python/test_poplar_kge_dataset.py:48-138), on the datasets of the committed fixtures
(tests/golden/sampler_*.npz, drawn with the reference's own generator): every sampled positive
decodes to a triple of the training set, `remote` is sorted, unique and zero-padded, labels are
where the exchange puts the positive tails; plus determinism and training straight from it."""

from pathlib import Path

import numpy as np
import pytest

from distributed_kge_poplar_b200 import capi, poplar_kge as kge
from helpers import BATCH_KEYS, check_batch_decodes_to_training_triples, engine_settings
from oracle.step_oracle import StepConfig

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).parent / "golden"


def _engine(f, n_step=3, **extra):
    n, B, a2a = int(f["n_shard"]), int(f["batch_size"]), int(f["a2a_size"])
    n_entity = int(f["shard_to_count"].max()) + 1
    n_rel = int(f["train_hrt"][:, 1].max()) + 1
    n_rel += (-n_rel) % n
    cfg = StepConfig(n_shard=n, n_entity=n_entity, n_relation_type=n_rel, embedding_size=16, entity_feature_size=0,
                     batch_size=B, a2a_size=a2a, score_fn="TransE", distance_fn="L1", gamma=4.0)
    engine = capi.CEngine(engine_settings(cfg, n_step=n_step, **extra))
    data = kge.Engine.bucket_triples(f["train_hrt"], f["entity_to_shard"], f["entity_to_idx"], n)
    engine.run("load_triples", dict(shard_to_count=np.ascontiguousarray(f["shard_to_count"], dtype=np.uint32), **data))
    return cfg, engine


def _sample(engine, cfg, n_step, seed):
    n, B, T = cfg.n_shard, cfg.batch_size, cfg.n_tail
    out = dict(remote=np.zeros((n, n_step, B + T), np.uint32), a2a=np.zeros((n, n_step, n, cfg.a2a_size), np.uint32),
               head=np.zeros((n, n_step, B), np.uint32), relation=np.zeros((n, n_step, B), np.uint32), tail=np.zeros((n, n_step, B), np.uint32))
    engine.run("sample_batch", dict(sample_seed=np.array([seed], np.uint32), **out))
    return out


@pytest.mark.parametrize("case", ["demo", "mid"])
def test_sampled_batches_decode_to_training_triples(case):
    f = np.load(GOLDEN / f"sampler_{case}.npz")
    cfg, engine = _engine(f)
    n, B = cfg.n_shard, cfg.batch_size
    seen = set()
    for run in range(4):
        batch = _sample(engine, cfg, 3, seed=11)
        check_batch_decodes_to_training_triples(batch, n, B, f["train_hrt"], f["entity_to_shard"], f["entity_to_idx"])
        # the labels are fixed: positive j of tail shard t sits in column t * a2a + j (src/python/poplar_kge_dataset.py:257-263)
        np.testing.assert_array_equal(batch["tail"], np.broadcast_to(f["batch0/tail"][:, :1], batch["tail"].shape))
        # every lookup names a gathered slot, negatives are real rows of their shard
        assert batch["head"].max() < B + cfg.n_tail and batch["a2a"].max() < B + cfg.n_tail
        for s in range(n):
            assert batch["remote"][s].max() <= f["shard_to_count"][s]
        seen.add(batch["remote"].tobytes())
    assert len(seen) == 4  # successive runs draw different batches
    engine.close()
    # the same seed on a fresh engine repeats the same sequence; another seed does not
    _, again = _engine(f)
    first = _sample(again, cfg, 3, seed=11)
    _, other = _engine(f)
    np.testing.assert_array_equal(first["remote"].tobytes() in seen, True)
    assert _sample(other, cfg, 3, seed=12)["remote"].tobytes() not in seen
    again.close()
    other.close()


def test_training_on_device_sampled_batches_matches_training_on_their_copy():
    """"train_step_loop_sampled" (no index array crosses the host) gives the loss and the state
    that "train_step_loop" gives on a host copy of the same sampled streams."""
    f = np.load(GOLDEN / "sampler_mid.npz")
    cfg, sampled = _engine(f)
    _, hosted = _engine(f)
    sampled.run("initialise_entities", {})
    hosted.run("initialise_entities", {})
    n = cfg.n_shard
    lr = np.full(n, 1e-2, np.float32)
    for run in range(2):
        batch = _sample(hosted, cfg, 3, seed=5)   # draws run `run` of seed 5 and leaves it staged; copy it back
        loss_host, loss_dev = np.zeros(n, np.float32), np.zeros(n, np.float32)
        hosted.run("train_step_loop", dict(learning_rate=lr, loss=loss_host, **batch))
        sampled.run("train_step_loop_sampled", dict(sample_seed=np.array([5], np.uint32), learning_rate=lr, loss=loss_dev))
        np.testing.assert_array_equal(loss_dev, loss_host)
        assert np.all(np.isfinite(loss_dev))
    rel_a, rel_b = (np.zeros((cfg.n_relation_type, cfg.embedding_size), np.float32) for _ in range(2))
    sampled.run("read", {"value": rel_a}, name="relation_embedding")
    hosted.run("read", {"value": rel_b}, name="relation_embedding")
    np.testing.assert_array_equal(rel_a, rel_b)
    sampled.close()
    hosted.close()


def test_sampler_argument_errors():
    f = np.load(GOLDEN / "sampler_demo.npz")
    cfg, engine = _engine(f)
    data = kge.Engine.bucket_triples(f["train_hrt"], f["entity_to_shard"], f["entity_to_idx"], cfg.n_shard)
    counts = np.ascontiguousarray(f["shard_to_count"], dtype=np.uint32)
    empty = {**data, "bucket_count": data["bucket_count"].copy()}
    empty["bucket_count"][0, 0] = 0
    with pytest.raises(ValueError, match="empty"):
        engine.run("load_triples", dict(shard_to_count=counts, **empty))
    with pytest.raises(ValueError, match="Key not found 'sample_seed'"):
        engine.run("sample_batch", {})
    fresh = capi.CEngine(engine_settings(cfg, n_step=3))
    with pytest.raises(RuntimeError, match="load_triples"):
        fresh.run("sample_batch", dict(sample_seed=np.array([1], np.uint32)))
    fresh.close()
    engine.close()
