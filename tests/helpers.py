"""Shared pieces of the tests: settings for both sides, seeded state and batches."""

from __future__ import annotations

from typing import Dict, Optional

import numpy as np

from oracle.step_oracle import Oracle, StepConfig

BATCH_KEYS = ("remote", "a2a", "head", "relation", "tail")


def engine_settings(cfg: StepConfig, n_step: int = 1, dtype: str = "float32",
                    feature_dtype: Optional[str] = None, rw_batch: int = 64, cuda_graph: bool = True,
                    seed: int = 1, **extra) -> Dict[str, object]:
    """The flattened settings dictionary the engine reads, from an oracle configuration."""
    s = {
        "model.seed": seed, "model.score_fn": cfg.score_fn, "model.distance_fn": cfg.distance_fn,
        "model.n_shard": cfg.n_shard, "model.n_entity": cfg.n_entity,
        "model.n_relation_type": cfg.n_relation_type, "model.embedding_size": cfg.embedding_size,
        "model.entity_feature_size": cfg.entity_feature_size, "model.feature_mlp_size": int(cfg.feature_mlp_size),
        "model.feature_dropout": float(cfg.feature_dropout), "model.share_feature_networks": cfg.share_feature_networks,
        "model.gamma": float(cfg.gamma), "model.init_scale": 1.0,
        "model.negative_adversarial_scale": float(cfg.negative_adversarial_scale),
        "training.adam_beta_m": cfg.adam_beta_m, "training.adam_beta_v": cfg.adam_beta_v,
        "training.adam_epsilon": cfg.adam_epsilon, "training.weight_decay": float(cfg.weight_decay),
        "training.learning_rate_modifiers": dict(cfg.learning_rate_modifiers),
        "data.batch_size": cfg.batch_size, "data.a2a_size": cfg.a2a_size,
        "training.loss.type": cfg.loss_type, "training.loss_scale": float(cfg.loss_scale),
        "training.embedding_regularisation.power": float(cfg.embedding_regularisation[0]),
        "training.embedding_regularisation.weight": float(cfg.embedding_regularisation[1]),
        "training.feature_regularisation.power": float(cfg.feature_regularisation[0]),
        "training.feature_regularisation.weight": float(cfg.feature_regularisation[1]),
        "training.hidden_regularisation.power": float(cfg.hidden_regularisation[0]),
        "training.hidden_regularisation.weight": float(cfg.hidden_regularisation[1]),
        "execution.device": "cuda", "execution.dtype": dtype,
        "execution.train_steps_per_program_run": n_step, "execution.rw_batch_size": rw_batch,
        "execution.predict_hr_batch_size": 8, "execution.predict_tail_batch_size": 64,
        "execution.predict_n_best": 5, "execution.cuda_graph": cuda_graph,
    }
    if cfg.loss_type == "softmax":
        s["training.loss.correction_weight"] = float(cfg.correction_weight)
    if feature_dtype is not None:
        s["execution.feature_dtype"] = feature_dtype
    s.update(extra)
    return s


def random_state(cfg: StepConfig, seed: int, fp16_features: bool = False, warm: bool = False):
    """Seeded initial state in float32: embeddings ~ N(0, 1/sqrt(d)), small dense parameters.

    ``warm`` also fills the optimiser state (as after some training), which exercises the
    sqrt(v) storage and the momentum terms instead of Adam's sign-like first step."""
    rng = np.random.RandomState(seed)
    d, f = cfg.embedding_size, cfg.entity_feature_size
    rows = np.zeros((cfg.n_shard, cfg.n_entity, cfg.row_size), np.float32)
    rows[..., :d] = rng.normal(size=rows[..., :d].shape) / np.sqrt(d)
    if f:
        feat = rng.normal(size=(cfg.n_shard, cfg.n_entity, f))
        if fp16_features:
            feat = feat.astype(np.float16)
        rows[..., 3 * d :] = feat.astype(np.float32)
        rows[:, 0, 3 * d :] = 0
    state = {"entity_data": rows, "step": np.zeros(cfg.n_shard, np.uint32)}
    if cfg.score_fn == "RotatE":  # one angle per complex pair
        state["relation_embedding"] = rng.uniform(-np.pi, np.pi, size=(cfg.n_relation_type, d // 2)).astype(np.float32)
    else:
        state["relation_embedding"] = (rng.normal(size=(cfg.n_relation_type, d)) / np.sqrt(d)).astype(np.float32)
    for name in cfg.projection_names:
        state[name] = (rng.normal(size=(f, d)) / np.sqrt(max(f, 1)) / np.sqrt(d)).astype(np.float32)
    dense_names = ("relation_embedding",) + cfg.projection_names
    if cfg.feature_mlp_size > 0:
        mrng, m = np.random.RandomState(seed + 104729), cfg.feature_mlp_size
        for name in cfg.projection_names:
            prefix = name[: -len("feature_projection")]
            state[prefix + "mlp_up_projection"] = (mrng.normal(size=(2 * d, m)) / np.sqrt(2 * d)).astype(np.float32)
            state[prefix + "mlp_down_projection"] = (mrng.normal(size=(m, d)) / np.sqrt(m)).astype(np.float32)
            dense_names += (prefix + "mlp_up_projection", prefix + "mlp_down_projection")
    if cfg.score_fn == "TransH":  # hyperplane normals, normalised on use
        state["relation_normal"] = (np.random.RandomState(seed + 7919).normal(size=(cfg.n_relation_type, d)) / np.sqrt(d)).astype(np.float32)
        dense_names += ("relation_normal",)
    for name in dense_names:
        state[name + "/adam_m"] = np.zeros_like(state[name])
        state[name + "/adam_v"] = np.zeros_like(state[name])
    if warm:
        scale = float(cfg.loss_scale) * 1e-3
        rows[..., d : 2 * d] = scale * rng.normal(size=rows[..., :d].shape)
        rows[..., 2 * d : 3 * d] = np.abs(scale * rng.normal(size=rows[..., :d].shape)) + 0.1 * scale
        for name in dense_names:
            state[name + "/adam_m"] = (scale * rng.normal(size=state[name].shape)).astype(np.float32)
            state[name + "/adam_v"] = ((scale * rng.normal(size=state[name].shape)) ** 2 + (0.1 * scale) ** 2).astype(np.float32)
        state["step"][:] = 37
    return state


def random_batch(cfg: StepConfig, n_step: int, seed: int, fixed_remote: bool = False,
                 pad: int = 0) -> Dict[str, np.ndarray]:
    """Index streams under the stream contract: ``remote`` rows unique, sorted, non-zero, then
    ``pad`` zeros (as the sampler's unique_pad leaves them); lookups avoid the padded slots."""
    rng = np.random.RandomState(seed)
    n, R = cfg.n_shard, cfg.n_remote
    used = R - pad
    remote = np.zeros((n, n_step, R), np.uint32)
    for s in range(n):
        for i in range(n_step):
            remote[s, i, :used] = np.sort(rng.permutation(np.arange(1, cfg.n_entity))[:used])
    if fixed_remote:
        remote[...] = remote[:, :1]
    u32 = lambda hi, shape: rng.randint(hi, size=shape).astype(np.uint32)  # noqa: E731
    return dict(remote=remote, a2a=u32(used, (n, n_step, n, cfg.a2a_size)),
                head=u32(used, (n, n_step, cfg.batch_size)),
                relation=u32(cfg.n_relation_type, (n, n_step, cfg.batch_size)),
                tail=u32(cfg.n_tail, (n, n_step, cfg.batch_size)))


def write_state(engine, cfg: StepConfig, state: Dict[str, np.ndarray], rw_batch: int,
                dtype=np.float32, shards: slice = slice(None)) -> None:
    """Load a state dictionary into a capi.CEngine through "write" and "write_entity_rows"."""
    for name, value in state.items():
        if name == "entity_data":
            continue
        engine.run("write", {"value": np.ascontiguousarray(value)}, name=name)
    rows = state["entity_data"][shards]
    n_local = rows.shape[0]
    for offset in range(0, cfg.n_entity, rw_batch):
        idx = np.arange(offset, offset + rw_batch, dtype=np.uint32)
        idx[idx >= cfg.n_entity] = 0
        chunk = rows[:, offset : offset + rw_batch]
        if chunk.shape[1] < rw_batch:
            # overflow slots point at row 0; give them row 0's data so the order does not matter
            fill = np.repeat(rows[:, :1], rw_batch - chunk.shape[1], axis=1)
            chunk = np.concatenate([chunk, fill], axis=1)
        engine.run("write_entity_rows", {
            "write_indices": np.ascontiguousarray(np.broadcast_to(idx, (n_local, rw_batch))),
            "write_data": np.ascontiguousarray(chunk.astype(dtype)),
        })


def read_rows(engine, cfg: StepConfig, rw_batch: int, n_local: int, dtype=np.float32) -> np.ndarray:
    out = []
    for offset in range(0, cfg.n_entity, rw_batch):
        idx = np.arange(offset, offset + rw_batch, dtype=np.uint32)
        idx[idx >= cfg.n_entity] = 0
        data = np.zeros((n_local, rw_batch, cfg.row_size), dtype)
        engine.run("read_entity", {
            "read_indices": np.ascontiguousarray(np.broadcast_to(idx, (n_local, rw_batch))),
            "read_data": data,
        })
        out.append(data[:, : cfg.n_entity - offset])
    return np.concatenate(out, axis=1)


def read_state(engine, cfg: StepConfig, rw_batch: int, n_local: int) -> Dict[str, np.ndarray]:
    state = {}
    for name, shape in engine.variables().items():
        value = np.zeros(shape, np.uint32 if name == "step" else np.float32)
        engine.run("read", {"value": value}, name=name)
        state[name] = value
    state["entity_data"] = read_rows(engine, cfg, rw_batch, n_local)
    return state


def make_oracle(cfg: StepConfig, state: Dict[str, np.ndarray], dtype=np.float64, seed: int = 1) -> Oracle:
    """`seed` is the engine's model.seed: with dropout on, the oracle is handed the engine's masks."""
    oracle = Oracle(cfg, dtype)
    oracle.set_state(state)
    if cfg.feature_dropout > 0:
        oracle.dropout_mask = lambda step, part: dropout_keep_mask(seed, step, part, cfg.n_shard, cfg.n_remote,
                                                                   cfg.embedding_size, cfg.feature_dropout)
    return oracle


def assert_close(actual, expected, rtol: float, what: str, atol_scale: float = 1.0) -> None:
    """|actual - expected| <= rtol * (|expected| + atol_scale * typical magnitude of the tensor).

    The magnitude term absorbs entries that are sums with heavy cancellation, whose own size
    says nothing about the rounding error of the terms they were summed from."""
    actual, expected = np.asarray(actual, np.float64), np.asarray(expected, np.float64)
    assert actual.shape == expected.shape, f"{what}: shape {actual.shape} != {expected.shape}"
    scale = float(np.sqrt(np.mean(expected**2))) if expected.size else 0.0
    err = np.abs(actual - expected)
    bound = rtol * (np.abs(expected) + atol_scale * scale) + 1e-30
    worst = np.unravel_index(np.argmax(err / bound), err.shape) if err.size else ()
    assert np.all(err <= bound), (
        f"{what}: max violation at {worst}: actual {actual[worst]!r} expected {expected[worst]!r} "
        f"(rtol {rtol}, tensor rms {scale:.3g})")


def philox_4x32_10(counter, key0: int, key1: int):
    """Philox-4x32 with ten rounds on four uint64 arrays holding 32-bit counters; returns the four words."""
    mask = np.uint64(0xFFFFFFFF)
    c = [np.asarray(x, np.uint64) & mask for x in counter]
    k0, k1 = np.uint64(key0 & 0xFFFFFFFF), np.uint64(key1 & 0xFFFFFFFF)
    m0, m1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
    for _ in range(10):
        p0, p1 = m0 * c[0], m1 * c[2]  # 32 x 32 -> 64 bit products
        hi0, lo0, hi1, lo1 = p0 >> np.uint64(32), p0 & mask, p1 >> np.uint64(32), p1 & mask
        c = [hi1 ^ c[1] ^ k0, lo1, hi0 ^ c[3] ^ k1, lo0]
        k0 = (k0 + np.uint64(0x9E3779B9)) & mask
        k1 = (k1 + np.uint64(0xBB67AE85)) & mask
    return c


def dropout_keep_mask(seed: int, step: int, part: int, n_shard: int, n_rows: int, d: int, p: float) -> np.ndarray:
    """Numpy restatement of the engine's dropout mask (csrc/kernels.cuh, dropout_keep4): bool
    [n_shard, n_rows, d], True where the element of gathered row r, column c is kept in training
    step `step` (counted from 1) by call `part` (0 head, 1 tail)."""
    threshold = int(round((1.0 - p) * 16777216.0))
    quads = (d + 3) // 4
    shard = np.arange(n_shard, dtype=np.uint64)[:, None, None]
    r = np.arange(n_rows, dtype=np.uint64)[None, :, None]
    q = np.arange(quads, dtype=np.uint64)[None, None, :]
    shape = (n_shard, n_rows, quads)
    words = philox_4x32_10([np.broadcast_to(r, shape), np.broadcast_to(q, shape), np.broadcast_to((shard << np.uint64(1)) | np.uint64(part), shape),
                            np.full(shape, 0x64726F70, np.uint64)], seed, step)
    keep = np.stack([(w >> np.uint64(8)) < threshold for w in words], axis=-1)  # [n, R, quads, 4]
    return keep.reshape(n_shard, n_rows, quads * 4)[:, :, :d]


def philox_normal4(seed: int, stream: int, row: np.ndarray, col4: np.ndarray) -> np.ndarray:
    """Numpy restatement of the engine's counter-based normal generator (csrc/kernels.cuh,
    philox_normal4): Philox-4x32-10 keyed by (seed, stream), counted by (row, column / 4), then two
    Box-Muller pairs.  Returns [..., 4] float64 for broadcast ``row`` / ``col4`` arrays."""
    row, col4 = np.broadcast_arrays(np.asarray(row, np.uint64), np.asarray(col4, np.uint64))
    c = philox_4x32_10([row, col4, np.full(row.shape, stream, np.uint64), np.full(row.shape, 0x6B676562, np.uint64)],
                       seed, 0x9E3779B9 ^ stream)
    u = [((x >> np.uint64(8)).astype(np.float64) + 0.5) / 16777216.0 for x in c]
    r0, r1 = np.sqrt(-2.0 * np.log(u[0])), np.sqrt(-2.0 * np.log(u[2]))
    a0, a1 = 2.0 * np.pi * u[1], 2.0 * np.pi * u[3]
    return np.stack([r0 * np.cos(a0), r0 * np.sin(a0), r1 * np.cos(a1), r1 * np.sin(a1)], axis=-1)


def expected_initial_table(seed: int, shard: int, n_rows: int, d: int, f: int, stddev: float) -> np.ndarray:
    """What "initialise_entities" leaves in a shard: [n_rows, 3d + f] float64 (value ~ N(0, stddev),
    zero optimiser state, features ~ N(0, 1) from a second stream, zero features in row 0)."""
    rows = np.arange(n_rows)[:, None]
    out = np.zeros((n_rows, 3 * d + f))
    value = philox_normal4(seed, shard, rows, np.arange((d + 3) // 4)[None, :]).reshape(n_rows, -1)[:, :d]
    out[:, :d] = stddev * value
    if f:
        feat = philox_normal4(seed ^ 0x5BD1E995, shard, rows, np.arange((f + 3) // 4)[None, :]).reshape(n_rows, -1)[:, :f]
        feat[0] = 0
        out[:, 3 * d:] = feat
    return out


def check_batch_decodes_to_training_triples(batch: Dict[str, np.ndarray], n_shard: int, batch_size: int, train_hrt, entity_to_shard,
                                            entity_to_idx) -> None:
    """The invariants of the reference's sampler tests (tests/python/test_poplar_kge_dataset.py:48-138)
    on index streams [n_shard, steps, ...]: following remote -> a2a -> exchange -> tail recovers an
    (h, r, t) of the training set for every positive, and `remote` is sorted, unique, zero-padded."""
    from oracle.step_oracle import all_to_all

    train = {tuple(t) for t in np.asarray(train_hrt).tolist()}
    lookup = {(int(s), int(i)): e for e, (s, i) in enumerate(zip(entity_to_shard, entity_to_idx))}
    remote, a2a, head, rel, tail = (np.asarray(batch[k]).astype(np.int64) for k in BATCH_KEYS)
    n = n_shard
    assert remote.shape[0] == n
    for step in range(remote.shape[1]):
        sent = np.stack([remote[s, step][a2a[s, step]] for s in range(n)])  # [src, dst, a2a]
        received = all_to_all(sent)  # [dst, src, a2a]
        for s in range(n):
            tails_local = received[s].reshape(-1)
            tail_shard = np.repeat(np.arange(n), a2a.shape[-1])
            for i in range(batch_size):
                h = lookup[(s, int(remote[s, step][head[s, step, i]]))]
                col = tail[s, step, i]
                t = lookup[(int(tail_shard[col]), int(tails_local[col]))]
                assert (h, int(rel[s, step, i]), t) in train
            row = remote[s, step]
            used = row[row > 0]
            assert np.all(np.diff(used) > 0) and np.all(row[len(used):] == 0)
