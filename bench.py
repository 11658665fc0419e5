"""Throughput of the BESS training step on 1..8 B200s: one JSON line on stdout.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload: the full-scale configuration (TransE-L2, d=256 fp32 embeddings and Adam state, 768
fp16 features through a learned 768x256 projection, 512 positives and 256 shared negatives per
shard, sampled-softmax loss) with one shard per GPU and 11 375 001 rows per shard: 91 M entities
at 8 GPUs, the same table per GPU at fewer (weak scaling; 91 M rows do not fit below 4 GPUs).
Inputs are synthetic with the shapes of WikiKG90Mv2: entity ids Zipf(1.1) over a fixed
pseudo-random permutation, relations Zipf(1.3), positives bucketed by (head shard, tail shard).

One bench "step" is one program run of the engine: 100 training steps on pre-staged index
arrays, the unit the reference's host loop works in (scripts/run_profile.py:43-51).
  value  device time of K program runs with the batch already on the GPU (CUDA events on the
         engine's stream), max over ranks
  e2e    wall time of K calls of the public "train_step_loop" command with host arrays:
         validation, host->device copy of the five index streams, segment preparation, the
         steps, device->host copy of the loss
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

ROWS_PER_SHARD = 11_375_001  # ceil(91 000 000 / 8) + the padding row
N_RELATION = 1387
BATCH, NEGATIVES, D, F = 512, 256, 256, 768
DEVICE_STEPS = 100
ENTITY_ALPHA, RELATION_ALPHA = 1.1, 1.3  # Zipf exponents of the synthetic ids; None = uniform
MODEL = {"score_fn": "TransE", "distance_fn": "L2", "loss": "softmax", "value_dtype": None, "feature_dtype": "float16",
         "title": "BESS TransE-L2 training", "precision": "d=256 fp32 + 768 fp16 features"}

# The training workloads of bench.py: "train" is the metric configuration (BASELINE configuration 3);
# "config4" is BASELINE configuration 4 (DistMult, d = 512, bf16 embedding values with fp32 Adam
# state, 1024 positives + 1024 shared negatives per shard, 30 M entities over 8 shards, 1000
# relations, uniform ids, no entity features), whose scores are bf16 tensor-core contractions.
WORKLOADS = {
    "train": {},
    "config4": dict(ROWS_PER_SHARD=3_750_001, N_RELATION=1000, BATCH=1024, NEGATIVES=1024, D=512, F=0, ENTITY_ALPHA=None,
                    RELATION_ALPHA=None,
                    MODEL={"score_fn": "DistMult", "distance_fn": "MatMul", "loss": "logsigmoid", "value_dtype": "bfloat16",
                           "feature_dtype": None, "title": "BESS DistMult training",
                           "precision": "d=512 bf16 values + fp32 Adam state, no features"}),
}


def select_workload(name: str) -> None:
    globals().update(WORKLOADS[name])


# ---------------------------------------------------------------------------
# Synthetic workload


def workload_settings(n_shard: int, rows_per_shard: int, device_steps: int, rank: int = 0, world: int = 1,
                      cuda_graph: bool = True) -> dict:
    n_rel = int(n_shard * np.ceil(N_RELATION / n_shard))
    a2a = (BATCH + NEGATIVES) // n_shard
    settings = {
        "model.seed": 2, "model.score_fn": MODEL["score_fn"], "model.distance_fn": MODEL["distance_fn"], "model.n_shard": n_shard,
        "model.n_entity": rows_per_shard, "model.n_relation_type": n_rel, "model.embedding_size": D,
        "model.entity_feature_size": F, "model.feature_mlp_size": 0, "model.feature_dropout": 0.0,
        "model.share_feature_networks": True, "model.gamma": 10.0, "model.init_scale": 1.0,
        "model.negative_adversarial_scale": 0.0,
        "training.adam_beta_m": 0.9, "training.adam_beta_v": 0.999, "training.adam_epsilon": 1e-8,
        "training.weight_decay": 0.0, "training.learning_rate_modifiers": {},
        "data.batch_size": BATCH, "data.a2a_size": a2a,
        "training.loss.type": MODEL["loss"], "training.loss.correction_weight": 1.0,
        "training.loss_scale": float(BATCH * n_shard * a2a),
        "training.embedding_regularisation.power": 3.0, "training.embedding_regularisation.weight": 0.0,
        "training.feature_regularisation.power": 3.0, "training.feature_regularisation.weight": 0.0,
        "training.hidden_regularisation.power": 3.0, "training.hidden_regularisation.weight": 0.0,
        "execution.device": "cuda", "execution.dtype": "float32",
        "execution.train_steps_per_program_run": device_steps, "execution.rw_batch_size": 512,
        "execution.predict_hr_batch_size": 128, "execution.predict_tail_batch_size": 1024,
        "execution.predict_n_best": 100, "execution.cuda_graph": cuda_graph,
        "execution.rank": rank, "execution.world_size": world, "execution.device_ordinal": rank if world > 1 else 0,
    }
    if MODEL["feature_dtype"]:
        settings["execution.feature_dtype"] = MODEL["feature_dtype"]
    if MODEL["value_dtype"]:
        settings["execution.value_dtype"] = MODEL["value_dtype"]
    return settings


def _bounded_zipf(rng: np.random.RandomState, alpha: float, limit: int, size: int) -> np.ndarray:
    """Ranks in [0, limit) with P(k) ~ (k+1)^-alpha, by rejecting the unbounded sampler's tail."""
    out = np.empty(0, np.int64)
    while out.size < size:
        draw = rng.zipf(alpha, size=int((size - out.size) * 1.4) + 16)
        out = np.concatenate([out, draw[draw <= limit] - 1])
    return out[:size]


class TriplePool:
    """Synthetic training triples, bucketed by (head shard, tail shard) as the reference's
    dataset index does (src/python/poplar_kge_dataset.py:199-241).

    Entity popularity is Zipf(1.1) over a fixed affine permutation of the ids; an entity's shard
    is ``id % n_shard`` and its row ``id // n_shard + 1`` (row 0 is the padding row), the divmod
    layout of src/python/poplar_kge_dataset.py:184-189.  Every rank builds the same pool from the
    same seed, so no data moves between processes."""

    def __init__(self, n_shard: int, rows_per_shard: int, n_relation: int, pool_size: int, seed: int = 2):
        rng = np.random.RandomState(seed)
        self.n_shard, self.rows = n_shard, rows_per_shard
        n_entity = n_shard * (rows_per_shard - 1)
        mult = 2_654_435_761 % n_entity
        while np.gcd(mult, n_entity) != 1:
            mult += 1
        permute = lambda k: (k * mult + 12_345) % n_entity  # noqa: E731
        draw = lambda alpha, limit: (_bounded_zipf(rng, alpha, limit, pool_size) if alpha else  # noqa: E731
                                     rng.randint(limit, size=pool_size).astype(np.int64))
        head = permute(draw(ENTITY_ALPHA, n_entity))
        tail = permute(draw(ENTITY_ALPHA, n_entity))
        rel = draw(RELATION_ALPHA, n_relation)
        pair = (head % n_shard) * n_shard + (tail % n_shard)
        order = np.argsort(pair, kind="stable")
        self.h = (head[order] // n_shard + 1).astype(np.uint32)
        self.t = (tail[order] // n_shard + 1).astype(np.uint32)
        self.r = rel[order].astype(np.uint32)
        counts = np.bincount(pair, minlength=n_shard * n_shard)
        self.count = counts.reshape(n_shard, n_shard)
        self.offset = np.concatenate([[0], np.cumsum(counts)[:-1]]).reshape(n_shard, n_shard)
        if np.any(self.count == 0):
            raise RuntimeError("triple pool too small: an empty (head shard, tail shard) bucket")

    def sample(self, n_step: int, batch: int, a2a: int, seed: int) -> dict:
        """Index streams [n_shard, n_step, ...] for every shard: the layout of the reference's
        ``Dataset.sample_batch`` (src/python/poplar_kge_dataset.py:310-393)."""
        n, rng = self.n_shard, np.random.RandomState(seed)
        pos = batch // n
        neg = a2a - pos
        pick = self.offset[:, None, :, None] + rng.randint(1 << 62, size=(n, n_step, n, pos)) % self.count[:, None, :, None]
        h, r, t = self.h[pick], self.r[pick], self.t[pick]  # [head shard, step, tail shard, pos]
        t_neg = (1 + rng.randint(1 << 62, size=(n, n_step, n, neg)) % (self.rows - 1)).astype(np.uint32)
        # rows shard s must gather: its heads, the positive tails it owns, the negatives it serves
        wanted = np.concatenate([h.reshape(n, n_step, -1),
                                 t.transpose(2, 1, 0, 3).reshape(n, n_step, -1),
                                 t_neg.transpose(2, 1, 0, 3).reshape(n, n_step, -1)], axis=2)
        width = wanted.shape[2]
        remote = np.zeros((n, n_step, width), np.uint32)
        lookup = np.zeros((n, n_step, width), np.uint32)
        for s in range(n):
            for i in range(n_step):
                unique, inverse = np.unique(wanted[s, i], return_inverse=True)
                remote[s, i, : unique.size] = unique
                lookup[s, i] = inverse
        a2a_idx = np.concatenate([lookup[:, :, batch : 2 * batch].reshape(n, n_step, n, pos),
                                  lookup[:, :, 2 * batch :].reshape(n, n_step, n, neg)], axis=3)
        tail = (np.arange(pos)[None, :] + a2a * np.arange(n)[:, None]).reshape(-1)
        return dict(remote=remote, a2a=np.ascontiguousarray(a2a_idx),
                    head=np.ascontiguousarray(lookup[:, :, :batch]),
                    relation=np.ascontiguousarray(r.reshape(n, n_step, batch)),
                    tail=np.ascontiguousarray(np.broadcast_to(tail.astype(np.uint32), (n, n_step, batch))))


def exchange_handles(blob: bytes, world: int) -> bytes:
    """All-gather of the engines' connection handles over the default process group, in rank order."""
    import torch.distributed as dist

    handles = [None] * world
    dist.all_gather_object(handles, blob)
    return b"".join(handles)


def local_slice(batch: dict, rank: int, world: int) -> dict:
    """The shards of one process: n_shard / world consecutive shards starting at rank * that."""
    n = batch["remote"].shape[0] // world
    return {k: np.ascontiguousarray(v[rank * n : (rank + 1) * n]) for k, v in batch.items()}


# ---------------------------------------------------------------------------
# Clocks


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index, self.lines, self.proc = gpu_index, [], None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        threading.Thread(target=self._read, daemon=True).start()

    def _read(self) -> None:
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, sm_max, power, reasons = [], [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                sm_max.append(float(parts[2]))
                power.append(float(parts[3]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[5:9]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(sm_max) if sm_max else None,
                "power_w": float(np.median(power)) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


# ---------------------------------------------------------------------------
# Algorithmic traffic of one training step of one shard (bytes), per kernel


def step_traffic(n_shard: int) -> dict:
    """Algorithmic bytes per launch, by the name the engine times the kernel under."""
    B, T = BATCH, BATCH + NEGATIVES
    R = B + T
    n_rel = int(n_shard * np.ceil(N_RELATION / n_shard))
    row_state, row_feat = (D * 2 if MODEL["value_dtype"] == "bfloat16" else D * 4) + 2 * D * 4, F * 2
    return {
        # the row gather: R whole rows out of the table, written once to the compact copy
        "gather": 2 * R * (row_state + row_feat),
        # reads value + features of R rows and the projection, writes the hidden rows
        "hidden": R * (D * 4 + row_feat) + F * D * 4 + R * D * 4,
        "route": 2 * (T + B) * D * 4 + B * D * 4,
        "score": (B + T) * D * 4 + B * T * 4,
        "loss": 2 * B * T * 4,
        "score_bwd": 2 * B * T * 4 + 2 * (B + T) * D * 4,
        # reads the lookup gradients and value/m/sqrt(v) of R rows, writes them back + hidden grads
        "entity_update": (B + T) * D * 4 + 2 * R * row_state + R * D * 4,
        "projection_bwd": R * row_feat + R * D * 4 + F * D * 4,
        "dense_partial": n_rel * D * 4 + B * D * 4,
        "dense_update": 5 * (n_rel + F) * D * 4,
        # the step as the reference's host sees it: gather R whole rows, scatter their state back
        "step": R * (row_state + row_feat) + R * row_state,
    }


def step_flops() -> dict:
    """Algorithmic floating-point operations per launch of the kernels that are bound by arithmetic:
    2 per multiply-add of the contraction as the reference states it (the three TF32 products that
    make up one fp32 product on the tensor cores count once), 3 per pair-element of the L2 distance."""
    B, T = BATCH, BATCH + NEGATIVES
    R = B + T
    return {
        "hidden": 2 * R * F * D,
        "projection_bwd": 2 * R * F * D,
        "score_bwd": 2 * (2 * B * T * D),
        "score": (2 if MODEL["distance_fn"] == "MatMul" else 3) * B * T * D,
    }


# Which unit bounds each kernel (the rest move bytes): the contractions run on the tensor cores,
# the direct L2 distance on the FP32 pipe.
# dram__bytes_read.sum + dram__bytes_write.sum per launch from an ncu capture of the same kernels on a
# small table (the step's kernels touch the same rows whatever the table size).
NCU_TRAFFIC: dict = {
    "train": {"hidden": 7_043_328, "projection_bwd": 8_984_832, "score_bwd": 5_841_408, "score": 1_329_408,
              "loss": 1_612_800, "entity_update": 8_143_360},
    "config4": {"score_bwd": 7_416_832, "score": 3_221_760, "loss": 8_430_592, "entity_update": 32_069_376},
}

TENSOR_KERNELS = ("hidden", "projection_bwd", "score_bwd")
FP32_KERNELS = ("score",)
FP32_PEAK_TFLOPS = 148 * 128 * 2 * 1.965e9 / 1e12  # FMA lanes x 2 x the maximum SM clock: nominal, not measured


def summarise_exchange_trace(flat: np.ndarray) -> dict:
    """Mean timeline of one step from the engine's optional hand-over stamps (KGE_EXCHANGE_TRACE=1),
    in microseconds after the end of the wait for the dense parameters (the start of `hidden`)."""
    t = np.asarray(flat, np.float64).reshape(256, 4, 3)
    kinds = ["tails", "tail_grads", "dense_partials", "dense_params"]
    rows = []
    for e in range(256):
        prev = t[(e - 1) % 256]
        if (t[e] > 0).all() and (prev > 0).all() and t[e, 0, 0] > prev[3, 2]:
            origin = prev[3, 2]  # the previous step's parameters have arrived: hidden begins
            if t[e, 3, 2] - origin < 1e4:
                rows.append((t[e] - origin).reshape(-1))
    if not rows:
        return {"steps": 0}
    mean = np.mean(rows, axis=0).reshape(4, 3)
    out = {"steps": len(rows)}
    for k, name in enumerate(kinds):
        out[name] = {"published": round(mean[k, 0], 2), "wait_began": round(mean[k, 1], 2), "wait_ended": round(mean[k, 2], 2)}
    return out


NVLINK_PEAK_GBS = {"nominal_per_direction": 900.0, "measured_peer_copy": 770.0}


def nvlink_block(trace: dict, n_shard: int) -> dict:
    """What crosses NVLink per GPU and step in each of the four hand-overs, and the rate it implies
    over the interval from the producer's publication to the end of the consumer's wait (the engine's
    stamps).  The payload of a hand-over has been stored by the producing kernel before it publishes,
    so this interval is the flag's flight plus the consumer's polling: a latency, and the rate is the
    one a step of this size can reach, far below the links' bandwidth."""
    T, n_rel = BATCH + NEGATIVES, int(n_shard * np.ceil(N_RELATION / n_shard))
    away = (n_shard - 1) / n_shard
    payload = {
        "tails": 2 * T * D * 4 * away,                      # rows and their lower TF32 plane
        "tail_grads": T * D * 4 * away,
        "dense_partials": (n_rel + F) * D * 4 * away,        # each row to the process that owns it
        "dense_params": ((n_rel + 2 * F) * D * 4 / n_shard) * (n_shard - 1),  # owned rows (+ lower plane of W) to every other replica
    }
    out = {"steps_traced": trace.get("steps", 0), "peak_gbs": NVLINK_PEAK_GBS, "bytes_per_gpu_step": sum(payload.values())}
    for name, nbytes in payload.items():
        if name not in trace:
            continue
        us = trace[name]["wait_ended"] - trace[name]["published"]
        entry = {"bytes": nbytes, "published_us": trace[name]["published"], "wait_ended_us": trace[name]["wait_ended"]}
        if us > 0:
            entry["gb_per_s"] = nbytes / (us * 1e-6) / 1e9
            entry["frac_of_900"] = entry["gb_per_s"] / NVLINK_PEAK_GBS["nominal_per_direction"]
        out[name] = entry
    return out


# ---------------------------------------------------------------------------
# Arms


def measured_peaks() -> dict:
    """HBM copy bandwidth and dense bf16 tensor throughput measured on this pool's B200s (the sustained
    figure: the kernels here are timed inside a long step), or the stated fallbacks."""
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        peaks = json.loads(path.read_text())
        return {"hbm_gbs": float(peaks["hbm_gbs"]), "tensor_tflops": float(peaks["bf16_tflops_sustained"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "tensor_tflops": 1400.0, "source": "fallback"}


class CpuArm:
    """The C++ / OpenMP restatement of the step (oracle/csrc/bess_step.cpp) on the host cores, on the
    GPU arm's configuration: same shards, same rows per shard, same per-step shapes.  The table is
    allocated untouched (zero pages that cost nothing until used) and only the rows that the sampled
    batches name are filled with seeded values, so set-up does not scale with the table.  If the
    host cannot map the table, the row count is halved until it can, and the sample text says so."""

    def __init__(self, n_shard: int, rows: int):
        from oracle import build as oracle_build
        from oracle.cpp_oracle import CppOracle
        from oracle.step_oracle import StepConfig

        oracle_build.build()
        self.n_shard, self.asked_rows = n_shard, rows
        self.a2a = (BATCH + NEGATIVES) // n_shard
        n_rel = int(n_shard * np.ceil(N_RELATION / n_shard))
        while True:
            cfg = StepConfig(n_shard=n_shard, n_entity=rows, n_relation_type=n_rel, embedding_size=D, entity_feature_size=F,
                             batch_size=BATCH, a2a_size=self.a2a, score_fn=MODEL["score_fn"], distance_fn=MODEL["distance_fn"],
                             gamma=10.0, loss_type=MODEL["loss"], correction_weight=1.0 if MODEL["loss"] == "softmax" else 0.0)
            try:
                self.oracle = CppOracle(cfg)
                break
            except MemoryError:
                rows = rows // 2 + 1
        self.rows = rows
        # all host cores, whatever OMP_NUM_THREADS a launcher has put into the environment
        self.oracle.set_threads(os.cpu_count() or 1)
        rng = np.random.RandomState(0)
        self.oracle.rel[0][...] = rng.normal(size=self.oracle.rel[0].shape) / D
        if F:
            self.oracle.proj[0][...] = rng.normal(size=self.oracle.proj[0].shape) / D / np.sqrt(F)
        pool = TriplePool(n_shard, rows, n_rel, max(200_000, 100_000 * n_shard * n_shard))
        self.batch = pool.sample(4, BATCH, self.a2a, seed=1)
        for s in range(n_shard):
            touched = np.unique(self.batch["remote"][s])
            block = np.zeros((touched.size, self.oracle.entity_data.shape[2]), np.float32)
            block[:, :D] = rng.normal(size=(touched.size, D)) / D
            if F:
                block[:, 3 * D:] = rng.normal(size=(touched.size, F)).astype(np.float16)
            self.oracle.entity_data[s, touched] = block
        self.steps_done = 0

    def run(self, seconds_target: float) -> dict:
        steps, start = 0, time.perf_counter()
        while True:
            i = self.steps_done % 4
            self.oracle.train_step(1e-3, *(np.ascontiguousarray(self.batch[k][:, i]) for k in ("remote", "a2a", "head", "relation", "tail")))
            steps += 1
            self.steps_done += 1
            elapsed = time.perf_counter() - start
            if elapsed >= seconds_target or steps >= 2000:
                break
        rows_note = f"{self.rows} rows per shard" + ("" if self.rows == self.asked_rows else f" (the host could not map {self.asked_rows})")
        return {"value": self.n_shard * BATCH * steps / elapsed, "unit": "triples/s", "cores": self.oracle.threads, "kind": "port",
                "seconds": elapsed,
                "sample": f"{steps} training steps of the C++/OpenMP restatement (oracle/csrc/bess_step.cpp), {self.n_shard} shard(s), "
                          f"same per-step shapes, {rows_note}, {elapsed:.1f} s"}


def cpu_baseline(seconds_target: float = 12.0, n_shard: int = 1, rows: int = ROWS_PER_SHARD) -> dict:
    out = CpuArm(n_shard, rows).run(seconds_target)
    out.pop("seconds")
    return out


def run_reference_arm(args) -> None:
    """The reference's CPU path is Poplar's CPU target, which needs the Poplar SDK: it cannot be
    installed here.  This arm times the oracle's C++/OpenMP port of the same step on the host cores,
    on the configuration of the GPU arm; one bench step is a bounded sample of about three seconds."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    n_shard = args.gpus
    arm = CpuArm(n_shard, args.rows_per_shard)
    results = []
    for i in range(args.warmup + args.steps):
        r = arm.run(3.0 if i >= args.warmup else 0.5)
        if i >= args.warmup:
            results.append(r)
    value = float(np.mean([r["value"] for r in results]))
    ms_per_step = 1e3 * float(np.mean([r.pop("seconds") for r in results]))
    line = {
        "impl": "reference", "metric": "train_triples_per_sec", "value": value, "unit": "triples/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(n_shard, arm.rows, DEVICE_STEPS),
        "cpu_baseline": {**results[-1], "value": value},
        "e2e": {"value": value, "unit": "triples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_config(n_shard: int, rows: int, device_steps: int, note: str = "") -> dict:
    cfg = {
        "workload": f"{MODEL['title']}, {n_shard} shard(s) x {rows} rows ({MODEL['precision']}), "
                    f"{BATCH} positives + {NEGATIVES} shared negatives per shard, {MODEL['loss']} loss, {device_steps} steps per program run",
        "n_shard": n_shard, "rows_per_shard": rows, "per_shard_batch": BATCH, "shared_negatives": NEGATIVES,
        "embedding_size": D, "feature_size": F, "steps_per_program_run": device_steps,
        "cache": "inputs larger than L2: one program run touches about 0.5 GB of distinct table rows",
    }
    if note:
        cfg["note"] = note
    return cfg


def run_ours(args) -> None:
    import torch
    import torch.distributed as dist

    from distributed_kge_poplar_b200 import capi

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE is {world}: launch with torch.distributed.run for N > 1")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the engine has no CPU path")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    if world > 1:
        # time stamps of the hand-overs between the processes (one thread per kernel writes three
        # words per hand-over): the source of the `nvlink` block
        os.environ["KGE_EXCHANGE_TRACE"] = "1"
    n_shard, rows, device_steps = world, args.rows_per_shard, args.device_steps
    settings = workload_settings(n_shard, rows, device_steps, rank, world, cuda_graph=not args.no_graph)
    settings["execution.device_ordinal"] = local_rank
    engine = capi.CEngine(settings)
    if world > 1:
        engine.comm_connect(exchange_handles(engine.comm_export(), world), world)
    engine.run("initialise_entities", {})
    rng = np.random.RandomState(2)
    n_rel = settings["model.n_relation_type"]
    engine.run("write", {"value": (rng.normal(size=(n_rel, D)) / D).astype(np.float32)}, name="relation_embedding")
    if F:
        engine.run("write", {"value": (rng.normal(size=(F, D)) / D / np.sqrt(F)).astype(np.float32)}, name="feature_projection")

    a2a = settings["data.a2a_size"]
    pool = TriplePool(n_shard, rows, n_rel, pool_size=max(400_000, 200_000 * n_shard * n_shard))
    batches = [local_slice(pool.sample(device_steps, BATCH, a2a, seed=100 + i), rank, world) for i in range(4)]
    lr = np.full(1, 1e-3, np.float32)
    loss = np.zeros(1, np.float32)
    h2d = sum(v.nbytes for v in batches[0].values()) + lr.nbytes
    triples_per_call = n_shard * BATCH * device_steps

    # -- value: device time of a program run, inputs resident in HBM ------------
    # Every run stages its batch again, so that the sort-and-segment preparation (part of the step:
    # the backward of the row gather) is inside the device-timed window; the upload of the index
    # streams is not (it belongs to e2e).
    for i in range(args.warmup):
        engine.stage_batch(batches[i % 4])
        engine.train_staged(1e-3, None)
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    device_ms, launches = 0.0, 0
    t0 = time.perf_counter()
    for i in range(args.steps):
        engine.stage_batch(batches[i % 4])
        engine.train_staged(1e-3, None)
        ms, n_launch = engine.last_run_stats()
        device_ms += ms
        launches += n_launch + 1
    barrier()
    wall_value = time.perf_counter() - t0
    device_s = max_over_ranks(device_ms / 1e3)
    value = triples_per_call * args.steps / device_s

    trace = None
    if world > 1 and rank == 0:
        trace = summarise_exchange_trace(engine.debug_fetch("exchange_trace", 0, 256 * 4 * 3))

    # -- e2e: the public command with host arrays ----------------------------
    for i in range(args.warmup):
        engine.run("train_step_loop", dict(learning_rate=lr, loss=loss, **batches[i % 4]))
    barrier()
    t0 = time.perf_counter()
    for i in range(args.steps):
        engine.run("train_step_loop", dict(learning_rate=lr, loss=loss, **batches[i % 4]))
    barrier()
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    clocks = sampler.stop() if rank == 0 else None
    final_loss = float(loss[0])

    # -- e2e with the batch sampler on the device: no index stream crosses the host ----------
    engine.run("load_triples", dict(triples=np.ascontiguousarray(np.stack([pool.h, pool.r, pool.t])),
                                    bucket_offset=pool.offset.astype(np.uint32), bucket_count=pool.count.astype(np.uint32),
                                    shard_to_count=np.full(n_shard, rows - 1, np.uint32)))
    seed = np.array([7], np.uint32)
    for i in range(args.warmup):
        engine.run("train_step_loop_sampled", dict(sample_seed=seed, learning_rate=lr, loss=loss))
    barrier()
    t0 = time.perf_counter()
    for i in range(args.steps):
        engine.run("train_step_loop_sampled", dict(sample_seed=seed, learning_rate=lr, loss=loss))
    barrier()
    sampled_s = max_over_ranks(time.perf_counter() - t0)

    # -- per-kernel times (plain launches bracketed by events), for the roofline ----
    engine.set_kernel_timing(True)
    engine.stage_batch(batches[0])
    for _ in range(2):
        engine.train_staged(1e-3, None)
    times = engine.kernel_times()
    engine.set_kernel_timing(False)
    engine.close()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    peaks = measured_peaks()
    peak = peaks["hbm_gbs"]
    traffic = step_traffic(n_shard)
    flops = step_flops()
    total_kernel_ms = sum(ms for ms, _ in times.values())
    kernels = {}
    for name, (ms, count) in sorted(times.items(), key=lambda kv: -kv[1][0]):
        per_launch_us = 1e3 * ms / max(count, 1)
        entry = {"share": ms / total_kernel_ms, "us_per_launch": per_launch_us, "launches": count}
        if name in traffic:
            entry["algorithmic_bytes"] = traffic[name]
            entry["gb_per_s"] = traffic[name] / (per_launch_us * 1e-6) / 1e9
        if name in flops:
            entry["algorithmic_flops"] = flops[name]
            entry["tflop_per_s"] = flops[name] / (per_launch_us * 1e-6) / 1e12
        kernels[name] = entry
    dominant = next(iter(kernels))
    dom = kernels[dominant]
    tensor_kernels = TENSOR_KERNELS + (("score",) if MODEL["distance_fn"] == "MatMul" else ())
    if dominant in tensor_kernels:
        roofline = {"bound": "tensor", "kernel": dominant, "achieved": dom["tflop_per_s"], "peak": peaks["tensor_tflops"],
                    "unit": "TFLOP/s", "frac": dom["tflop_per_s"] / peaks["tensor_tflops"], "peak_source": peaks["source"],
                    "peak_note": "dense bf16 sustained; " + ("bf16 products, fp32 accumulation" if MODEL["value_dtype"] == "bfloat16" and dominant in ("score", "score_bwd")
                                                             else "the kernel computes fp32 products as three TF32 products"),
                    "algorithmic_flops_per_launch": dom["algorithmic_flops"]}
    elif dominant in FP32_KERNELS and dominant not in tensor_kernels:
        roofline = {"bound": "fp32", "kernel": dominant, "achieved": dom["tflop_per_s"], "peak": FP32_PEAK_TFLOPS,
                    "unit": "TFLOP/s", "frac": dom["tflop_per_s"] / FP32_PEAK_TFLOPS, "peak_source": "nominal",
                    "algorithmic_flops_per_launch": dom["algorithmic_flops"]}
    else:
        achieved = dom.get("gb_per_s", 0.0)
        roofline = {"bound": "hbm", "kernel": dominant, "achieved": achieved, "peak": peak, "unit": "GB/s",
                    "frac": achieved / peak, "peak_source": peaks["source"],
                    "algorithmic_bytes_per_launch": dom.get("algorithmic_bytes")}
    step_us = 1e6 * device_s / (args.steps * device_steps)
    line = {
        "metric": "train_triples_per_sec", "value": value, "unit": "triples/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * device_s / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16" if MODEL["value_dtype"] == "bfloat16" else "f32", "data": "synthetic",
        "config": workload_config(n_shard, rows, device_steps),
        "e2e": {"value": triples_per_call * args.steps / e2e_s, "unit": "triples/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": loss.nbytes, "ms_per_step": 1e3 * e2e_s / args.steps},
        "e2e_device_sampler": {"value": triples_per_call * args.steps / sampled_s, "unit": "triples/s", "h2d_bytes_per_step": int(lr.nbytes + 4),
                               "d2h_bytes_per_step": loss.nbytes, "ms_per_step": 1e3 * sampled_s / args.steps,
                               "note": "\"train_step_loop_sampled\": positives, negatives, unique rows and routing indices are drawn on the GPU"},
        "gpu_launches": int(launches),
        "roofline": {**roofline, "traffic": NCU_TRAFFIC.get(args.workload, {}).get(dominant), "us_per_launch": dom["us_per_launch"],
                     "step_us": step_us, "step_hbm_gb_per_s": traffic["step"] / (step_us * 1e-6) / 1e9,
                     "step_frac_of_hbm": traffic["step"] / (step_us * 1e-6) / 1e9 / peak},
        "kernels": kernels,
        "clocks": clocks,
        "wall_ms_per_step_value_arm": 1e3 * wall_value / args.steps,
        "final_loss": final_loss,
    }
    if trace is not None:
        line["nvlink"] = nvlink_block(trace, n_shard)
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(rows=rows)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_micro(args) -> None:
    """BASELINE configuration 2: single kernels on one GPU, device-timed through the C ABI's microbenchmark
    entry points.  Row gather and row-wise Adam scatter over R unique rows of a 2 000 000-row table of
    [value | adam_m | sqrt(adam_v)] (3 x 256 fp32 per row), ids Zipf(1.1) over a random permutation,
    seed 1; scores of 4096 (h, r) queries against 256 shared negative tails, d = 256, as L1, L2 (FP32
    pipe), dot product and L2 in contraction form (tensor cores).  CPU baseline: the reference's own
    l1dist / l2dist (oracle/_ref, compiled from its codelet sources) where built, on a bounded sample."""
    import ctypes

    import torch

    from distributed_kge_poplar_b200 import capi

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the engine has no CPU path")
    rows, d, queries, tails = 2_000_000, 256, 4096, 256
    rng = np.random.RandomState(1)
    perm = rng.permutation(rows)
    peaks = measured_peaks()
    sampler = ClockSampler(0)
    sampler.start()
    gathers, scatters = [], []
    for n in (4096, 16384, 65536, 262144, 1048576):
        ranks = _bounded_zipf(rng, 1.1, rows, n)
        idx = np.unique(perm[ranks]).astype(np.uint32)   # what the sampler's unique_pad leaves of n draws
        state_bytes = idx.size * 3 * d * 4
        g_us = capi.microbench_rows(0, rows, d, idx, max(args.steps, 5))
        s_us = capi.microbench_rows(1, rows, d, idx, max(args.steps, 5))
        scatter_bytes = 2 * state_bytes + 2 * idx.size * d * 4   # state in and out, gradient row in, hidden gradient out
        gathers.append({"draws": n, "rows": int(idx.size), "us": g_us, "gb_per_s": 2 * state_bytes / g_us / 1e3,
                        "frac_of_hbm": 2 * state_bytes / g_us / 1e3 / peaks["hbm_gbs"]})
        scatters.append({"draws": n, "rows": int(idx.size), "us": s_us, "gb_per_s": scatter_bytes / s_us / 1e3,
                         "frac_of_hbm": scatter_bytes / s_us / 1e3 / peaks["hbm_gbs"]})
    scores = {}
    for fn, name, flop in ((0, "l1_fp32_pipe", 3), (1, "l2_fp32_pipe", 3), (2, "dot_tensor_3xtf32", 2), (3, "l2_tensor_3xtf32", 2)):
        us = capi.microbench_scores(fn, queries, tails, d, max(10 * args.steps, 50))
        tf = flop * queries * tails * d / us / 1e6
        peak = peaks["tensor_tflops"] if fn >= 2 else FP32_PEAK_TFLOPS
        scores[name] = {"us": us, "pairs_per_s": queries * tails / us * 1e6, "tflop_per_s": tf, "peak_tflops": peak, "frac": tf / peak}
    clocks = sampler.stop()
    best = max(gathers, key=lambda g: g["gb_per_s"])
    line = {
        "metric": "microbench_gather_gb_per_s", "value": best["gb_per_s"], "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "higher_is_better": True, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"single kernels: gather / Adam scatter of R rows out of {rows} x (3 x {d} fp32), ids Zipf(1.1) seed 1; "
                               f"{queries} x {tails} scores, d = {d}"},
        "roofline": {"bound": "hbm", "kernel": "k_gather_step_rows", "achieved": best["gb_per_s"], "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": best["gb_per_s"] / peaks["hbm_gbs"], "peak_source": peaks["source"],
                     "algorithmic_bytes_per_launch": 2 * best["rows"] * 3 * d * 4, "traffic": None},
        "gather": gathers, "adam_scatter": scatters, "scores": scores, "clocks": clocks,
    }
    # the reference's own distance code on the host cores (one pair per call, as its vertex computes them)
    ref_path = ROOT / "oracle" / "_ref" / "libref_distance.so"
    if ref_path.exists() and not args.no_cpu_baseline:
        lib = ctypes.CDLL(str(ref_path))
        fp = ctypes.POINTER(ctypes.c_float)
        a = rng.normal(size=(64, d)).astype(np.float32)
        b = rng.normal(size=(tails, d)).astype(np.float32)
        base = {}
        for name in ("ref_l1dist", "ref_l2dist"):
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = ctypes.c_float, [fp, fp, ctypes.c_size_t]
            pa = [row.ctypes.data_as(fp) for row in a]
            pb = [row.ctypes.data_as(fp) for row in b]
            t0 = time.perf_counter()
            for x in pa:
                for y in pb:
                    fn(x, y, d)
            base[name] = len(pa) * len(pb) / (time.perf_counter() - t0)
        line["cpu_baseline"] = {"value": base["ref_l2dist"], "unit": "pairs/s", "cores": 1, "kind": "reference",
                                "sample": f"64 x {tails} pairs, d = {d}, of the reference's l2dist (and l1dist: {base['ref_l1dist']:.3g} pairs/s) "
                                          "compiled from its codelet sources, one call per pair through ctypes"}
    print(json.dumps(line), flush=True)


def run_predict(args) -> None:
    """BASELINE configuration 5: sharded ranking.  1250 (h, r) queries per GPU (10 000 over 8) are
    scored by TransE-L2, d = 256 fp32, against every row of every shard (11 375 001 rows per GPU, fp16
    features through the learned projection), each shard keeps its 100 best per query and the lists go
    back to the asking shard's process; the host merges them to a global top 10.  One bench step =
    one such ranking of 1250 queries per GPU."""
    import torch
    import torch.distributed as dist

    from distributed_kge_poplar_b200 import capi

    rank, world, local_rank = (int(os.environ.get(k, "0")) for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"))
    world = max(world, 1)
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE is {world}: launch with torch.distributed.run for N > 1")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the engine has no CPU path")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    rows = args.rows_per_shard or ROWS_PER_SHARD
    hr, n_best, queries_per_gpu = 1250, 100, 1250   # one pass over the table serves all of a GPU's queries
    settings = workload_settings(world, rows, 1, rank, world)
    settings.update({"execution.predict_hr_batch_size": hr, "execution.predict_n_best": n_best, "execution.device_ordinal": local_rank})
    engine = capi.CEngine(settings)
    if world > 1:
        engine.comm_connect(exchange_handles(engine.comm_export(), world), world)
    engine.run("initialise_entities", {})
    rng = np.random.RandomState(4)
    n_rel = settings["model.n_relation_type"]
    engine.run("write", {"value": (rng.normal(size=(n_rel, D)) / D).astype(np.float32)}, name="relation_embedding")
    engine.run("write", {"value": (rng.normal(size=(F, D)) / D / np.sqrt(F)).astype(np.float32)}, name="feature_projection")
    mult = 2_654_435_761 % (rows - 1)
    heads = (1 + (_bounded_zipf(rng, 1.1, rows - 1, queries_per_gpu) * mult + 12_345) % (rows - 1)).astype(np.uint32)
    rels = _bounded_zipf(rng, 1.3, N_RELATION, queries_per_gpu).astype(np.uint32)
    count = np.full(1, rows - 1, np.uint32)
    scores = np.zeros((1, world, hr, n_best), np.float32)
    indices = np.zeros((1, world, hr, n_best), np.uint32)

    def rank_all():
        best = np.zeros((queries_per_gpu, 10), np.float32)
        for lo in range(0, queries_per_gpu, hr):
            engine.run("predict", dict(predict_head=np.ascontiguousarray(heads[None, lo:lo + hr]), predict_relation=np.ascontiguousarray(rels[None, lo:lo + hr]),
                                       predict_entity_count=count, predict_scores=scores, predict_indices=indices))
            merged = scores[0].transpose(1, 0, 2).reshape(hr, -1)   # [query, shard * n_best]: the global top 10 on the host
            best[lo:lo + hr] = -np.sort(-merged, axis=1)[:, :10]
        return best

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    for _ in range(max(1, args.warmup // 3)):
        rank_all()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    t0 = time.perf_counter()
    launches = 0
    for _ in range(args.steps):
        best = rank_all()
        launches += engine.last_run_stats()[1] * (queries_per_gpu // hr)
    barrier()
    seconds = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([seconds], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        seconds = float(t.item())
    clocks = sampler.stop() if rank == 0 else None
    engine.close()
    if rank == 0:
        per_step = seconds / args.steps
        pairs = queries_per_gpu * world * (rows - 1) * world   # every query against every row of every shard
        flop = pairs * (2 * D) + (rows - 1) * world * 2 * F * D * (queries_per_gpu // hr)  # scores + hidden rows of every pass
        peaks = measured_peaks()
        print(json.dumps({
            "metric": "ranked_queries_per_sec", "value": queries_per_gpu * world / per_step, "unit": "queries/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": 1e3 * per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"sharded ranking: {queries_per_gpu} queries per GPU against {world} x {rows - 1} rows, TransE-L2 d={D}, "
                                   f"{F} fp16 features, per-shard top {n_best} in passes of {hr} queries, global top 10 on the host"},
            "e2e": {"value": queries_per_gpu * world / per_step, "unit": "queries/s", "h2d_bytes_per_step": int(2 * 4 * queries_per_gpu),
                    "d2h_bytes_per_step": int(2 * scores.nbytes * (queries_per_gpu // hr))},
            "gpu_launches": int(launches),
            "roofline": {"bound": "tensor", "kernel": "k_tc_planes (hidden rows and L2 scores of a pass)", "achieved": flop / per_step / world / 1e12,
                         "peak": peaks["tensor_tflops"], "unit": "TFLOP/s", "frac": flop / per_step / world / 1e12 / peaks["tensor_tflops"],
                         "peak_source": peaks["source"], "traffic": None,
                         "algorithmic_flops_per_step": flop, "peak_note": "dense bf16 sustained; fp32 products run as three TF32 products"},
            "clocks": clocks, "best_score_of_first_query": float(best[0, 0]),
        }), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS) + ["micro", "predict"], default="train",
                    help="train: the metric configuration; config4: DistMult with bf16 values; micro: single kernels (configuration 2); "
                         "predict: sharded ranking (configuration 5)")
    ap.add_argument("--rows-per-shard", type=int, default=None, help="smaller tables for profiler captures")
    ap.add_argument("--device-steps", type=int, default=DEVICE_STEPS, help="training steps per program run")
    ap.add_argument("--no-graph", action="store_true", help="launch kernel by kernel instead of replaying a CUDA graph")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.workload == "micro":
        return run_micro(args)
    if args.workload == "predict":
        return run_predict(args)
    select_workload(args.workload)
    if args.rows_per_shard is None:
        args.rows_per_shard = ROWS_PER_SHARD
    if args.warmup < 3 and args.impl == "ours" and args.rows_per_shard == ROWS_PER_SHARD:
        args.warmup = 3
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
