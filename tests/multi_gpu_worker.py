"""One rank of the multi-GPU parity check; started by tests/test_multi_gpu.py under torch.distributed.run.

Four shards on two processes (two local shards each), so rows travel both through local memory
and into the peer GPU's memory.  Every rank compares its slices with the float64 oracle."""

import os
import sys
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[1]
sys.path[:0] = [str(ROOT), str(ROOT / "tests")]


def main() -> None:
    import torch
    import torch.distributed as dist

    import bench
    from distributed_kge_poplar_b200 import capi
    from helpers import BATCH_KEYS, assert_close, engine_settings, make_oracle, random_batch, random_state, read_state, write_state
    from oracle.step_oracle import StepConfig

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local_rank = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    variant = sys.argv[1] if len(sys.argv) > 1 else "l2"
    kw = dict(score_fn="TransE", distance_fn="L2", loss_type="softmax", correction_weight=1.0, gamma=10.0)
    if variant == "distmult":
        kw = dict(score_fn="DistMult", distance_fn="MatMul", loss_type="logsigmoid")
    if variant == "transh":  # the step of separate kernels with a fourth dense parameter (the normals)
        kw = dict(score_fn="TransH", distance_fn="L1", loss_type="logsigmoid", gamma=6.0)
    if variant == "mlp":  # more dense parameters (the MLP's projections, pushed to their owners), dropout masks per global shard, regularisers
        kw = dict(score_fn="TransE", distance_fn="L2", loss_type="softmax", correction_weight=1.0, gamma=10.0, feature_dropout=0.25,
                  hidden_regularisation=(2.0, 0.02), feature_mlp_size=16)
    cfg = StepConfig(n_shard=2 * world, n_entity=400, n_relation_type=8, embedding_size=32, entity_feature_size=16,
                     batch_size=24, a2a_size=10, **kw)
    n_local, n_step, rw, lr = cfg.n_shard // world, 3, 64, 2e-3
    mine = slice(rank * n_local, (rank + 1) * n_local)
    state = random_state(cfg, 31, fp16_features=True, warm=True)
    engine = capi.CEngine(engine_settings(cfg, n_step=n_step, feature_dtype="float16", rw_batch=rw,
                                          **{"execution.rank": rank, "execution.world_size": world,
                                             "execution.device_ordinal": local_rank}))
    engine.comm_connect(bench.exchange_handles(engine.comm_export(), world), world)
    write_state(engine, cfg, state, rw, shards=mine)
    dist.barrier()
    oracle = make_oracle(cfg, state)
    for call in range(2):
        batch = random_batch(cfg, n_step, 40 + call, pad=3)
        want = oracle.train_step_loop(lr, batch)
        loss = np.zeros(n_local, np.float32)
        engine.run("train_step_loop", dict(learning_rate=np.full(n_local, lr, np.float32), loss=loss,
                                           **bench.local_slice(batch, rank, world)))
        assert_close(loss, want[mine], 1e-4, f"rank {rank} call {call}: loss", atol_scale=0)
    # No host barrier here on purpose: a run ends only when every process's share of the dense
    # update has arrived in this process's memory, so the state can be read straight away.
    got, ref = read_state(engine, cfg, rw, n_local), oracle.get_state()
    d = cfg.embedding_size
    assert_close(got["entity_data"][..., : 3 * d], ref["entity_data"][mine][..., : 3 * d], 1e-3 if variant == "transh" else 1e-4, f"rank {rank}: rows")
    # TransH's gradients are sums of signs (an L1 form): over six steps one rounding flip of a sign moves an entry visibly
    dense_tol = 1e-3 if variant == "transh" else 1e-4
    for key in ref:
        if key not in ("entity_data", "step"):
            assert_close(got[key], ref[key], dense_tol, f"rank {rank}: {key}")
    np.testing.assert_array_equal(got["step"], ref["step"])

    # ranking across processes, again with no host barrier since the training call
    hr, n_best = 8, 5
    rng = np.random.RandomState(9)
    head = (1 + rng.randint(cfg.n_entity - 1, size=(cfg.n_shard, hr))).astype(np.uint32)
    rel = rng.randint(cfg.n_relation_type, size=(cfg.n_shard, hr)).astype(np.uint32)
    counts = np.full(cfg.n_shard, cfg.n_entity - 1, np.uint32)
    scores = np.zeros((n_local, cfg.n_shard, hr, n_best), np.float32)
    rows = np.zeros(scores.shape, np.uint32)
    engine.run("predict", dict(predict_head=np.ascontiguousarray(head[mine]), predict_relation=np.ascontiguousarray(rel[mine]),
                               predict_entity_count=np.ascontiguousarray(counts[mine]), predict_scores=scores, predict_indices=rows))
    for l in range(n_local):
        s = rank * n_local + l
        q = np.stack([np.full(hr, s), head[s], rel[s]], axis=1)
        _, want_score = oracle.predict(q, counts, n_best)
        merged = -np.sort(-scores[l].transpose(1, 0, 2).reshape(hr, -1), axis=1)[:, :n_best]
        np.testing.assert_allclose(merged, want_score, rtol=1e-4, atol=1e-5)
    dist.barrier()

    # A rank that does not take part: the other rank's device-side wait gives up within seconds,
    # the call returns an error and the process goes on (nothing faults, nothing hangs).
    if variant == "l2":
        batch = bench.local_slice(random_batch(cfg, n_step, 50, pad=3), rank, world)
        if rank == 0:
            t0 = time.time()
            try:
                engine.run("train_step_loop", dict(learning_rate=np.full(n_local, lr, np.float32),
                                                   loss=np.zeros(n_local, np.float32), **batch))
                raise AssertionError("the lone rank's step should have reported the missing peer")
            except RuntimeError as e:
                assert "gave up" in str(e), str(e)
            assert time.time() - t0 < 60
            # this engine's hand-over epochs now disagree with its peer's: it refuses further work
            try:
                engine.run("train_step_loop", dict(learning_rate=np.full(n_local, lr, np.float32),
                                                   loss=np.zeros(n_local, np.float32), **batch))
                raise AssertionError("an engine whose wait gave up should refuse further steps")
            except RuntimeError as e:
                assert "must be rebuilt" in str(e), str(e)
        dist.barrier()
    engine.close()
    dist.barrier()
    print(f"MULTI_GPU_OK rank {rank} {variant}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
