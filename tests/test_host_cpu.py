"""Host-side checks that need no GPU: the shared library exports what the header declares,
settings errors carry the reference's texts, the host mirror of the reference's Python
interface behaves like it, and the benchmark's synthetic batches obey the stream contract."""

import re
from pathlib import Path

import numpy as np
import pytest

from distributed_kge_poplar_b200 import capi, poplar_kge as kge
from helpers import engine_settings
from oracle.step_oracle import StepConfig

ROOT = Path(__file__).resolve().parents[1]
CFG = StepConfig(n_shard=2, n_entity=50, n_relation_type=4, embedding_size=8, entity_feature_size=4,
                 batch_size=4, a2a_size=3)


def test_library_exports_every_declared_entry_point():
    header = (ROOT / "include" / "kge_b200.h").read_text()
    declared = set(re.findall(r"\b(kge_[a-z_0-9]+)\s*\(", header))
    declared -= {"kge_status", "kge_dtype", "kge_setting_type"}
    lib = capi.load_library()
    assert declared == set(capi.SYMBOLS)
    for name in declared:
        assert hasattr(lib, name), name


def test_settings_errors_precede_the_device():
    """Settings are parsed before any CUDA call, so these behave the same with or without a GPU
    (src/poplar_kge.cpp:39-67, 237-246, 294-300, 278-285, 586-591)."""
    good = engine_settings(CFG)
    with pytest.raises(ValueError, match="Key not found 'model.n_shard'"):
        capi.CEngine({k: v for k, v in good.items() if k != "model.n_shard"})
    with pytest.raises(ValueError, match="Key 'model.gamma' holds value of unexpected type"):
        capi.CEngine({**good, "model.gamma": 2})
    with pytest.raises(ValueError, match="'execution.dtype' must either be 'float16' or 'float32', not 'bfloat16'"):
        capi.CEngine({**good, "execution.dtype": "bfloat16"})
    with pytest.raises(ValueError, match="'model.score_fn' must be one of"):
        capi.CEngine({**good, "model.score_fn": "TransF"})
    with pytest.raises(ValueError, match="'model.distance_fn' must be one of"):
        capi.CEngine({**good, "model.distance_fn": "L3"})
    with pytest.raises(ValueError, match="'training.loss.type' must be one of 'logsigmoid' or 'softmax'"):
        capi.CEngine({**good, "training.loss.type": "hinge"})
    with pytest.raises(ValueError, match=r"Parameter 'relation_embedding' shape\[0\] \(5\) is not divisible by n_shard \(2\)"):
        capi.CEngine({**good, "model.n_relation_type": 5})
    with pytest.raises(ValueError, match="Bad training.learning_rate_modifier: unknown parameter 'nope'"):
        capi.CEngine({**good, "training.learning_rate_modifiers": {"nope": 2.0}})
    with pytest.raises(ValueError, match="Key not found 'training.loss.correction_weight'"):
        capi.CEngine({**good, "training.loss.type": "softmax"})
    with pytest.raises(ValueError, match="'model.feature_dropout' must be in"):
        capi.CEngine({**good, "model.feature_dropout": 1.0})
    with pytest.raises(ValueError, match="regularisation.power' must be at least 1"):
        capi.CEngine({**good, "training.hidden_regularisation.power": 0.5, "training.hidden_regularisation.weight": 0.1})


def test_attach_failure_is_a_runtime_error():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    with pytest.raises(RuntimeError, match="Could not attach"):  # the text the reference's tests skip on
        capi.CEngine(engine_settings(CFG))


def test_predictions_topk_and_sort():
    """tests/python/test_poplar_kge.py:15-45."""
    pre = kge.Predictions(
        shard_idx=np.array([[[10, 100], [20, 200], [30, 300], [40, 400]], [[50, 500], [60, 600], [70, 700], [80, 800]]]),
        score=np.array([[2, 1, 3, 0], [-4, -3, -2, -1]]))
    post = pre.topk(k=3).sort()
    np.testing.assert_equal(post.shard_idx, [[[30, 300], [10, 100], [20, 200]], [[80, 800], [70, 700], [60, 600]]])
    np.testing.assert_equal(post.score, [[3, 2, 1], [-1, -2, -3]])
    multi = kge.Predictions(pre.shard_idx[:, None], pre.score[:, None]).topk(k=3).sort()
    assert multi.shard_idx.shape == (2, 1, 3, 2) and multi.score.shape == (2, 1, 3)
    np.testing.assert_equal(multi.shard_idx[:, 0], post.shard_idx)


def test_settings_tree_matches_the_reference_layout():
    s = kge.Settings.create_demo()
    s.seed = 100
    s.prepare()
    flat = s.flatten()
    assert flat["model.n_shard"] == 2 and flat["data.a2a_size"] == 5 and flat["training.loss.type"] == "logsigmoid"
    assert flat["training.loss_scale"] == 6 * 2 * 5  # batch * n_shard * a2a (src/python/poplar_kge.py:259-262)
    assert s.n_tail == 10 and s.n_remote == 16 and s.entity_data_r_size == 30
    assert s.program_runs_per_log == 4 and s.logs_per_training_run == 5
    # seeds derive from the top-level seed exactly as the reference derives them
    children = np.random.SeedSequence(100).spawn(3)
    assert s.model.seed == int(children[0].generate_state(1)[0])
    assert s.data.seed == int(children[1].generate_state(1)[0])
    engine_keys = s.engine_settings()
    assert "logging.path" not in engine_keys and "code_changes" not in engine_keys
    assert all(v is not None for v in engine_keys.values())
    wiki = kge.Settings.create_wikikg90mv2(8).prepare()
    assert wiki.model.n_entity == 11403828 and wiki.model.n_relation_type == 1392 and wiki.n_remote == 1280


def test_reference_settings_agree_where_a_checkout_exists():
    from golden import reference_loader

    if not reference_loader.available():
        pytest.skip("no checkout of the reference")
    ref_kge, _, _ = reference_loader.load()
    ours, theirs = kge.Settings.create_demo(), ref_kge.Settings.create_demo()
    ours.seed = theirs.seed = 5
    a, b = ours.prepare().flatten(), theirs.prepare().flatten()
    for key, value in b.items():
        if key in ("code_changes", "execution.device"):
            continue
        assert a[key] == value, key


def test_benchmark_batches_obey_the_stream_contract():
    import bench

    n, rows, batch, a2a = 4, 5001, 64, 24
    pool = bench.TriplePool(n, rows, 8, 40_000)
    triples = set()
    for hs in range(n):
        for ts in range(n):
            lo, cnt = pool.offset[hs, ts], pool.count[hs, ts]
            for h, r, t in zip(pool.h[lo : lo + cnt], pool.r[lo : lo + cnt], pool.t[lo : lo + cnt]):
                triples.add((hs, int(h), int(r), ts, int(t)))
    b = pool.sample(3, batch, a2a, seed=9)
    remote, lookups, head, rel, tail = (b[k].astype(np.int64) for k in ("remote", "a2a", "head", "relation", "tail"))
    assert remote.shape == (n, 3, batch + n * a2a) and lookups.shape == (n, 3, n, a2a)
    for step in range(3):
        sent = np.stack([remote[s, step][lookups[s, step]] for s in range(n)])  # [src, dst, a2a]
        received = np.swapaxes(sent, 0, 1).reshape(n, n * a2a)
        for s in range(n):
            row = remote[s, step]
            used = row[row > 0]
            assert np.all(np.diff(used) > 0) and np.all(row[used.size :] == 0) and row.max() < rows
            for i in range(batch):
                col = tail[s, step, i]
                assert (s, int(row[head[s, step, i]]), int(rel[s, step, i]), col // a2a, int(received[s, col])) in triples
    sliced = bench.local_slice(b, rank=1, world=2)
    np.testing.assert_array_equal(sliced["remote"], b["remote"][2:4])


def test_exchange_trace_summary():
    """bench.summarise_exchange_trace: mean step timeline from the engine's hand-over stamps."""
    import bench

    t = np.zeros((256, 4, 3))
    for e in range(1, 200):  # epoch e: a step of 100 us that starts at 100 * e
        start = 100.0 * e
        t[e % 256] = [[start + 20, start + 21, start + 22], [start + 60, start + 61, start + 62],
                      [start + 90, start + 91, start + 92], [start + 99, start + 99.5, start + 100]]
    out = bench.summarise_exchange_trace(t.reshape(-1))
    assert out["steps"] >= 190
    assert abs(out["tails"]["published"] - 20) < 1e-6 and abs(out["dense_params"]["wait_ended"] - 100) < 1e-6
    assert bench.summarise_exchange_trace(np.zeros(256 * 4 * 3)) == {"steps": 0}


def test_predict_chunk_count_is_the_same_on_every_process():
    """Each engine "predict" call synchronises the processes, so the number of calls must not
    depend on which shards a process holds: it follows the longest per-shard query list over all
    shards (uneven counts: shard 3 has 70 queries, shard 0 has 2, shard 1 none)."""
    from distributed_kge_poplar_b200 import poplar_kge

    settings = poplar_kge.Settings.create_demo().prepare()
    settings.model.n_shard = 4
    settings.execution.predict_hr_batch_size = 30
    shards = np.array([0] * 2 + [2] * 31 + [3] * 70)

    class Holder:  # predict_chunks reads nothing but the settings
        pass

    counts = []
    for rank in range(4):
        holder = Holder()
        holder.settings = settings
        counts.append(poplar_kge.Engine.predict_chunks(holder, shards))
    assert counts == [3, 3, 3, 3]
    holder = Holder()
    holder.settings = settings
    assert poplar_kge.Engine.predict_chunks(holder, np.zeros(0, np.int64)) == 0
    assert poplar_kge.Engine.predict_chunks(holder, np.array([1] * 30)) == 1


def test_documented_switches_are_the_ones_the_sources_read():
    """Every KGE_* environment switch that the engine or the Python twin reads is described in the
    integration notes, and the notes describe no switch that nothing reads."""
    documented = set(re.findall(r"`(KGE_[A-Z0-9_]+)", (ROOT / "INTEGRATION.md").read_text()))
    read = set()
    for path in (ROOT / "distributed-kge-poplar_b200").rglob("*"):
        if path.suffix in (".cu", ".cuh", ".hpp", ".cpp", ".py"):
            text = path.read_text()
            read |= set(re.findall(r'getenv\("(KGE_[A-Z0-9_]+)"', text))
            read |= set(re.findall(r'environ(?:\.get)?\(?\[?"(KGE_[A-Z0-9_]+)"', text))
    assert read, "no switch found: the patterns above no longer match the sources"
    assert documented == read
