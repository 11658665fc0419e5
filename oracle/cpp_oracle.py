"""ctypes driver of oracle/csrc/bess_step.cpp (TEST INFRASTRUCTURE ONLY).

Holds the same state as ``step_oracle.Oracle`` in float32 and advances it with the compiled
C++ / OpenMP restatement of the step; used as the timed CPU baseline and as a second checker.
"""

from __future__ import annotations

import ctypes as C
from pathlib import Path
from typing import Dict

import numpy as np

from .step_oracle import StepConfig

LIB_PATH = Path(__file__).resolve().parent / "_build" / "libbess_oracle.so"

_SCORE = {"TransE": 0, "DistMult": 1, "ComplEx": 2}
_DIST = {"L1": 0, "L1_old": 0, "L2": 1, "L2_old": 1, "MatMul": 2}
_LOSS = {"logsigmoid": 0, "softmax": 1}


class _Config(C.Structure):
    _fields_ = [(k, C.c_int) for k in ("n_shard", "n_entity", "n_relation_type", "d", "f", "batch", "a2a",
                                       "score_fn", "dist_fn", "loss_fn", "share_networks")] + \
               [(k, C.c_float) for k in ("gamma", "correction_weight", "loss_scale", "beta_m", "beta_v",
                                         "epsilon", "weight_decay")]


def load():
    if not LIB_PATH.exists():
        raise ImportError(f"{LIB_PATH} is missing: run `python oracle/build.py`")
    lib = C.CDLL(str(LIB_PATH))
    fp, up = C.POINTER(C.c_float), C.POINTER(C.c_uint32)
    lib.bess_oracle_step.argtypes = [C.POINTER(_Config), fp, fp, fp, fp, fp, fp, fp, C.POINTER(C.c_uint), C.c_float,
                                     up, up, up, up, up, fp]
    lib.bess_oracle_threads.restype = C.c_int
    lib.bess_oracle_set_threads.argtypes = [C.c_int]
    lib.bess_oracle_set_threads.restype = None
    return lib


def _no_huge_pages(array: np.ndarray) -> None:
    """A table of many gigabytes is mapped untouched and only the rows a run names are ever written.
    With transparent huge pages every first touch would zero two megabytes; ordinary pages keep the
    cost of a touched row at a few kilobytes.  Best effort: ignored where madvise is not available."""
    try:
        libc = C.CDLL("libc.so.6", use_errno=True)
        page = 4096
        start = (array.ctypes.data + page - 1) // page * page
        length = (array.ctypes.data + array.nbytes - start) // page * page
        if length > 0:
            libc.madvise(C.c_void_p(start), C.c_size_t(length), 14 + 1)  # MADV_NOHUGEPAGE
    except OSError:
        pass


class CppOracle:
    def __init__(self, cfg: StepConfig):
        if cfg.negative_adversarial_scale or cfg.learning_rate_modifiers:
            raise ValueError("the C++ restatement does not cover adversarial weights or learning-rate modifiers")
        self.cfg, self.lib = cfg, load()
        self.c = _Config(cfg.n_shard, cfg.n_entity, cfg.n_relation_type, cfg.embedding_size, cfg.entity_feature_size,
                         cfg.batch_size, cfg.a2a_size, _SCORE[cfg.score_fn], _DIST[cfg.distance_fn], _LOSS[cfg.loss_type],
                         int(cfg.share_feature_networks), cfg.gamma, cfg.correction_weight, cfg.loss_scale,
                         cfg.adam_beta_m, cfg.adam_beta_v, cfg.adam_epsilon, cfg.weight_decay)
        d, f = cfg.embedding_size, cfg.entity_feature_size
        n_net = len(cfg.projection_names) if f else 0
        self.entity_data = np.zeros((cfg.n_shard, cfg.n_entity, cfg.row_size), np.float32)
        _no_huge_pages(self.entity_data)
        self.rel = [np.zeros((cfg.n_relation_type, d), np.float32) for _ in range(3)]
        self.proj = [np.zeros((max(n_net, 1), f, d), np.float32) for _ in range(3)]
        self.step = C.c_uint(0)

    @property
    def threads(self) -> int:
        return int(self.lib.bess_oracle_threads())

    def set_threads(self, n: int) -> None:
        self.lib.bess_oracle_set_threads(int(n))

    def set_state(self, state: Dict[str, np.ndarray]) -> None:
        self.entity_data[...] = state["entity_data"]
        for k, suffix in enumerate(("", "/adam_m", "/adam_v")):
            self.rel[k][...] = state["relation_embedding" + suffix]
            if self.cfg.entity_feature_size:
                for i, name in enumerate(self.cfg.projection_names):
                    self.proj[k][i] = state[name + suffix]
        (step,) = {int(s) for s in np.atleast_1d(state["step"])}
        self.step = C.c_uint(step)

    def get_state(self) -> Dict[str, np.ndarray]:
        out = {"entity_data": self.entity_data.copy(), "step": np.full(self.cfg.n_shard, self.step.value, np.uint32)}
        for k, suffix in enumerate(("", "/adam_m", "/adam_v")):
            out["relation_embedding" + suffix] = self.rel[k].copy()
            for i, name in enumerate(self.cfg.projection_names):
                out[name + suffix] = self.proj[k][i].copy() if self.cfg.entity_feature_size else np.zeros((0, self.cfg.embedding_size), np.float32)
        return out

    def train_step(self, lr: float, remote, a2a, head, relation, tail) -> np.ndarray:
        fp, up = C.POINTER(C.c_float), C.POINTER(C.c_uint32)
        idx = [np.ascontiguousarray(x, dtype=np.uint32) for x in (remote, a2a, head, relation, tail)]
        loss = np.zeros(self.cfg.n_shard, np.float32)
        f = lambda a: a.ctypes.data_as(fp)  # noqa: E731
        self.lib.bess_oracle_step(C.byref(self.c), f(self.entity_data), f(self.rel[0]), f(self.rel[1]), f(self.rel[2]),
                                  f(self.proj[0]), f(self.proj[1]), f(self.proj[2]), C.byref(self.step), lr,
                                  *(x.ctypes.data_as(up) for x in idx), f(loss))
        return loss

    def train_step_loop(self, lr: float, batch: Dict[str, np.ndarray]) -> np.ndarray:
        n_step = batch["remote"].shape[1]
        total = np.zeros(self.cfg.n_shard, np.float32)
        for i in range(n_step):
            total += self.train_step(lr, *(np.ascontiguousarray(batch[k][:, i]) for k in ("remote", "a2a", "head", "relation", "tail")))
        return total / np.float32(n_step)
