"""Generate the fixtures in this folder from the reference's own Python code.

Run where a checkout of the reference exists:  ``python tests/golden/make_golden.py``

* ``train_<case>.npz``: the reference's torch model (tests/python/reference_model.py)
  trained from a written-out initial state on cycled random batches with the
  ``remote`` rows held fixed, the protocol of tests/python/test_poplar_kge.py:175-259.
  Holds the settings, the initial state, the batches, the per-loop losses, the
  final state and the brute-force predictions after training.
* ``sampler_<case>.npz``: batches drawn by the reference's BESS sampler
  (src/python/poplar_kge_dataset.py:310-393) with the sharding tables needed to
  decode them: the routing / bucketing fixture.
"""

from __future__ import annotations

import dataclasses
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
import reference_loader  # noqa: E402


def make_settings(ref_kge, case: str):
    s = ref_kge.Settings.create_demo()
    s.seed = 100
    if case == "mid":
        s.seed = 7
        s.model.n_shard = 4
        s.model.n_entity = 200
        s.model.n_relation_type = 8
        s.model.embedding_size = 32
        s.model.entity_feature_size = 16
        s.model.gamma = 4.0
        s.data.batch_size = 32
        s.data.a2a_size = 12
        s.data.dataset.n_train = 400
        s.data.dataset.n_eval = 40
        s.training.learning_rate = 0.01
        s.training.n_step = 12
        s.logging.steps_per_log = 3
        s.execution.train_steps_per_program_run = 3
        s.execution.predict_n_best = 10
    s.prepare()
    return s


def random_batch(settings, rng: np.random.RandomState):
    """Random index arrays under the stream contract: unique, sorted, non-zero
    ``remote`` rows; everything else uniform (tests/python/test_poplar_kge.py:51-86
    states the same constraints)."""
    n, steps = settings.model.n_shard, settings.execution.train_steps_per_program_run
    remote = np.stack(
        [
            np.sort(rng.permutation(np.arange(1, settings.model.n_entity))[: settings.n_remote])
            for _ in range(n * steps)
        ]
    ).reshape(n, steps, settings.n_remote)
    u32 = lambda hi, shape: rng.randint(hi, size=shape).astype(np.uint32)  # noqa: E731
    return dict(
        remote=remote.astype(np.uint32),
        a2a=u32(settings.n_remote, (n, steps, n, settings.data.a2a_size)),
        head=u32(settings.n_remote, (n, steps, settings.data.batch_size)),
        relation=u32(settings.model.n_relation_type, (n, steps, settings.data.batch_size)),
        tail=u32(settings.n_tail, (n, steps, settings.data.batch_size)),
    )


def initial_state(settings, features: np.ndarray, rng: np.random.RandomState):
    """Same distributions as the reference's initialisation
    (src/python/poplar_kge.py:625-663, src/poplar_kge.cpp:864-871), written out so
    that no device RNG is involved."""
    m = settings.model
    scale = m.init_scale / m.embedding_size
    normal = lambda shape: rng.normal(size=shape).astype(np.float32)  # noqa: E731
    state = {
        "step": np.zeros(m.n_shard, np.uint32),
        "relation_embedding": scale * normal((m.n_relation_type, m.embedding_size)),
        "feature_projection": (scale / np.sqrt(m.entity_feature_size))
        * normal((m.entity_feature_size, m.embedding_size)),
    }
    for name in ("relation_embedding", "feature_projection"):
        state[name] = state[name].astype(np.float32)
        state[name + "/adam_m"] = np.zeros_like(state[name])
        state[name + "/adam_v"] = np.zeros_like(state[name])
    rows = np.zeros((m.n_shard, m.n_entity, settings.entity_data_r_size), np.float32)
    rows[:, :, : m.embedding_size] = scale * normal((m.n_shard, m.n_entity, m.embedding_size))
    rows[:, :, 3 * m.embedding_size :] = features.astype(np.float32)
    state["entity_data"] = rows
    return state


def flat_settings(settings) -> dict:
    out = {}
    for key, value in settings.flatten().items():
        if value is None or key in ("logging.path", "logging.predict_at", "code_changes"):
            continue
        out[key] = value
    return out


def make_training_case(ref_kge, ref_data, ref_model, case: str) -> None:
    import torch

    torch.manual_seed(0)
    settings = make_settings(ref_kge, case)
    data = ref_data.RawData.load(settings)
    dataset = ref_data.Dataset.load(data, settings)
    rng = np.random.RandomState(settings.model.seed)
    features = dataset.entity_features(settings.model.entity_feature_size)
    state0 = initial_state(settings, features, rng)
    model = ref_model.Model(settings)
    model.set_state(state0)
    reference_loader.fix_adam_step(model)

    batches = [random_batch(settings, rng) for _ in range(3)]
    for b in batches:
        b["remote"][...] = batches[0]["remote"][:, 0, np.newaxis, :]
    n_loop = settings.program_runs_per_log * settings.logs_per_training_run
    losses = []
    for i in range(n_loop):
        b = batches[i % 3]
        losses.append(model.train_step_loop(ref_kge.Batch(**b)))
    final = model.get_state()

    rng_q = np.random.RandomState(1234)
    n_query = 2 * settings.execution.predict_hr_batch_size + 3
    queries = np.stack(
        [
            rng_q.randint(settings.model.n_shard, size=n_query),
            1 + rng_q.randint(settings.model.n_entity - 1, size=n_query),
            rng_q.randint(settings.model.n_relation_type, size=n_query),
        ],
        axis=-1,
    ).astype(np.uint32)
    with torch.no_grad():
        pred = model.predict(queries, shard_to_count=dataset.shard_to_count)

    out = {f"settings/{k}": np.asarray(v) for k, v in flat_settings(settings).items() if not isinstance(v, dict)}
    out.update({f"initial/{k}": v for k, v in state0.items()})
    out.update({f"final/{k}": np.asarray(v) for k, v in final.items()})
    for i, b in enumerate(batches):
        out.update({f"batch{i}/{k}": v for k, v in b.items()})
    out["n_loop"] = np.asarray(n_loop)
    out["loss_mean_per_loop"] = np.asarray(losses, np.float64)
    out["shard_to_count"] = np.asarray(dataset.shard_to_count)
    out["predict/queries"] = queries
    out["predict/shard_idx"] = np.asarray(pred.shard_idx).astype(np.uint32)
    out["predict/score"] = np.asarray(pred.score, np.float32)
    np.savez_compressed(HERE / f"train_{case}.npz", **out)
    print(case, "losses", np.round(losses, 5))


def make_sampler_case(ref_kge, ref_data, case: str) -> None:
    settings = make_settings(ref_kge, case)
    data = ref_data.RawData.load(settings)
    dataset = ref_data.Dataset.load(data, settings)
    out = {}
    for i in range(2):
        b = dataset.sample_batch()
        out.update({f"batch{i}/{k}": np.asarray(v).astype(np.uint32) for k, v in dataclasses.asdict(b).items()})
    out["train_hrt"] = data.train_hrt
    out["entity_to_shard"] = dataset.entity_to_shard.astype(np.uint32)
    out["entity_to_idx"] = dataset.entity_to_idx.astype(np.uint32)
    out["shard_to_count"] = dataset.shard_to_count.astype(np.uint32)
    out["n_shard"] = np.asarray(settings.model.n_shard)
    out["batch_size"] = np.asarray(settings.data.batch_size)
    out["a2a_size"] = np.asarray(settings.data.a2a_size)
    np.savez_compressed(HERE / f"sampler_{case}.npz", **out)


def main() -> None:
    ref_kge, ref_data, ref_model = reference_loader.load()
    for case in ("demo", "mid"):
        make_training_case(ref_kge, ref_data, ref_model, case)
        make_sampler_case(ref_kge, ref_data, case)


if __name__ == "__main__":
    main()
