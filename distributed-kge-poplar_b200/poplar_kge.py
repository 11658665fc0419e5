"""Host-side interface of the B200 BESS engine, with the reference's names.

Mirrors the public surface of the reference's ``src/python/poplar_kge.py`` (the
``Settings`` tree :36-413, ``Batch`` :416-432, ``Predictions`` :435-468 and
``Engine`` :471-861) so that drivers written against it keep working: same class,
field and method names, same array shapes and dtypes, same exceptions.  The
engine underneath is the pybind11 module ``libpoplar_kge`` built from
``csrc/`` over the C ABI of ``include/kge_b200.h``.

Differences a caller can see:
  * ``execution.device`` may be "cuda"; the reference's "cpu"/"ipu" are taken to
    mean the GPU too, so existing settings run unchanged.
  * ``ExecutionSettings`` has optional extras (feature_dtype, device_ordinal, rank,
    world_size, cuda_graph); ``Engine`` takes ``rank``/``world_size`` and, when
    world_size > 1, an ``exchange`` callable that all-gathers a bytes object
    across the processes (one process per GPU).
  * ``Engine.write_entity_rows`` writes whole rows, optimiser state included.
  * ``Engine.dump`` / ``Engine.restore`` write and load a checkpoint with one file per shard.
  * ``Engine.load_triples`` / ``sample_batch`` / ``train_step_loop_sampled`` draw batches on the device.
"""

from __future__ import annotations

import dataclasses
import importlib.util
import json
import sys
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Callable, Dict, List, Optional, Sequence, Set, Tuple, Union

import numpy as np

_HERE = Path(__file__).resolve().parent
Shape = Tuple[int, ...]


def _load_engine_module():
    """Import the compiled ``libpoplar_kge`` that sits beside this file (no fallback)."""
    if "libpoplar_kge" in sys.modules and getattr(sys.modules["libpoplar_kge"], "Engine", None):
        return sys.modules["libpoplar_kge"]
    candidates = sorted(_HERE.glob("libpoplar_kge*.so"))
    if not candidates:
        raise ImportError(
            f"no libpoplar_kge*.so in {_HERE}: build it with `python distributed-kge-poplar_b200/build.py`")
    spec = importlib.util.spec_from_file_location("libpoplar_kge", candidates[0])
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    sys.modules["libpoplar_kge"] = module
    return module


# ---------------------------------------------------------------------------
# Settings


@dataclass
class ModelSettings:
    seed: Optional[int]
    score_fn: str  # TransE | DistMult | ComplEx
    distance_fn: str  # L1 | L2 | MatMul
    n_shard: int
    n_entity: int  # rows per shard, padding row 0 included
    n_relation_type: int
    embedding_size: int
    entity_feature_size: int
    feature_mlp_size: int
    feature_dropout: float
    negative_adversarial_scale: float
    share_feature_networks: bool
    gamma: float
    init_scale: float


@dataclass
class WikiKg90Mv2Settings:
    name: str = "wikikg90mv2"


@dataclass
class GeneratedDataSettings:
    n_train: int
    n_eval: int
    seed: Optional[int]
    name: str = "generated"


@dataclass
class CubicRootRelationSampling:
    type: str = "cubic_root"


@dataclass
class DataSettings:
    seed: Optional[int]
    dataset: Union[WikiKg90Mv2Settings, GeneratedDataSettings]
    batch_size: int  # positives per shard
    a2a_size: int  # rows sent to each peer shard
    entity_feature_mapping: str
    sampling_strategy: Optional[CubicRootRelationSampling]


@dataclass
class LinearLearningRateDecay:
    type: str = "linear"


@dataclass
class SteppedLearningRateDecay:
    step: int
    multiplier: float
    type: str = "stepped"


@dataclass
class ExponentialLearningRateDecay:
    half_life_steps: int
    type: str = "exponential"


@dataclass
class LogSigmoidLoss:
    type: str = "logsigmoid"


@dataclass
class SoftmaxLoss:
    correction_weight: float
    type: str = "softmax"


@dataclass
class NormRegularisation:
    power: float
    weight: float


@dataclass
class TrainingSettings:
    n_step: int
    validation_interval: int
    loss: Union[LogSigmoidLoss, SoftmaxLoss]
    embedding_regularisation: NormRegularisation
    feature_regularisation: NormRegularisation
    hidden_regularisation: NormRegularisation
    learning_rate: float
    learning_rate_decay: Union[None, LinearLearningRateDecay, SteppedLearningRateDecay,
                               ExponentialLearningRateDecay]
    learning_rate_modifiers: Dict[str, float]
    adam_beta_m: float
    adam_beta_v: float
    adam_epsilon: float
    weight_decay: float
    loss_scale: Optional[float]


@dataclass
class ExecutionSettings:
    device: str
    dtype: str  # "float32" | "float16": type of a table row and of the host arrays
    train_steps_per_program_run: int
    rw_batch_size: int
    predict_hr_batch_size: int
    predict_tail_batch_size: int
    predict_n_best: int
    feature_dtype: Optional[str] = None  # storage type of the feature part; default = dtype
    device_ordinal: Optional[int] = None
    rank: Optional[int] = None
    world_size: Optional[int] = None
    cuda_graph: Optional[bool] = None


@dataclass
class LogSettings:
    path: Optional[Path]
    wandb: bool
    steps_per_log: int
    predict_at: Tuple[float, ...]


def _zero_regulariser() -> NormRegularisation:
    return NormRegularisation(power=3.0, weight=0.0)


@dataclass
class Settings:
    seed: Optional[int]
    model: ModelSettings
    data: DataSettings
    training: TrainingSettings
    execution: ExecutionSettings
    logging: LogSettings
    code_changes: Tuple[str, ...] = ()

    # -- derived sizes -------------------------------------------------------

    def _ceil_ratio(self, numerator: float, *denominators: float) -> int:
        value = float(numerator)
        for d in denominators:
            value /= d
        return int(np.ceil(value))

    @property
    def program_runs_per_log(self) -> int:
        return self._ceil_ratio(self.logging.steps_per_log, self.execution.train_steps_per_program_run)

    @property
    def logs_per_training_run(self) -> int:
        return self._ceil_ratio(self.training.n_step, self.execution.train_steps_per_program_run,
                                self.program_runs_per_log)

    @property
    def logs_per_validation(self) -> int:
        return self._ceil_ratio(self.training.validation_interval,
                                self.execution.train_steps_per_program_run, self.program_runs_per_log)

    @property
    def n_tail(self) -> int:
        return self.model.n_shard * self.data.a2a_size

    @property
    def n_remote(self) -> int:
        return self.data.batch_size + self.n_tail

    @property
    def entity_data_r_size(self) -> int:
        return 3 * self.model.embedding_size + self.model.entity_feature_size

    @property
    def entity_data_r_shape(self) -> Shape:
        return (self.model.n_shard, self.execution.rw_batch_size, self.entity_data_r_size)

    @property
    def entity_data_w_shape(self) -> Shape:
        return (self.model.n_shard, self.execution.rw_batch_size, self.model.entity_feature_size)

    @property
    def predict_at_log(self) -> Set[int]:
        per_log = self.execution.train_steps_per_program_run * self.program_runs_per_log
        return {int(round(t * self.training.n_step / per_log)) for t in self.logging.predict_at}

    @property
    def relation_embedding_size(self) -> int:
        return self.model.embedding_size // 2 if self.model.score_fn == "RotatE" else self.model.embedding_size

    # -- preparation ---------------------------------------------------------

    def prepare(self) -> "Settings":
        """Fill in the seeds and the default loss scale (batch * n_shard * a2a)."""
        if self.seed is None:
            self.seed = int(np.random.randint(1 << 30))
        children = np.random.SeedSequence(self.seed).spawn(3)
        model_seed, data_seed, raw_seed = (int(c.generate_state(1)[0]) for c in children)
        if self.model.seed is None:
            self.model.seed = model_seed
        if self.data.seed is None:
            self.data.seed = data_seed
        if isinstance(self.data.dataset, GeneratedDataSettings) and self.data.dataset.seed is None:
            self.data.dataset.seed = raw_seed
        if isinstance(self.logging.path, str):
            self.logging.path = Path(self.logging.path)
        if self.training.loss_scale is None:
            self.training.loss_scale = float(self.data.batch_size * self.model.n_shard * self.data.a2a_size)
        return self

    def flatten(self) -> Dict[str, Any]:
        """Dotted-key view of the tree, e.g. ``{"model.n_shard": 8, ...}``."""
        flat: Dict[str, Any] = {}

        def walk(node: Any, path: Tuple[str, ...]) -> None:
            if dataclasses.is_dataclass(node):
                for name, child in vars(node).items():
                    walk(child, path + (name,))
            else:
                flat[".".join(path)] = node

        walk(self, ())
        return flat

    def engine_settings(self) -> Dict[str, Any]:
        """What is handed to the compiled engine: ``flatten()`` minus host-only keys and Nones."""
        skip = {"logging.path", "logging.predict_at", "code_changes"}
        return {k: v for k, v in self.flatten().items() if k not in skip and v is not None}

    # -- presets -------------------------------------------------------------

    @classmethod
    def create_demo(cls) -> "Settings":
        """A toy configuration: 2 shards x 90 rows, d=8, 6 features, TransE-L1."""
        return cls(
            seed=None,
            model=ModelSettings(seed=None, score_fn="TransE", distance_fn="L1", n_shard=2, n_entity=90,
                                n_relation_type=12, embedding_size=8, entity_feature_size=6,
                                feature_mlp_size=0, feature_dropout=0.0, negative_adversarial_scale=0.0,
                                share_feature_networks=True, gamma=2.0, init_scale=1.0),
            data=DataSettings(seed=None, dataset=GeneratedDataSettings(n_train=50, n_eval=50, seed=None),
                              batch_size=6, a2a_size=5, entity_feature_mapping="full",
                              sampling_strategy=CubicRootRelationSampling()),
            training=TrainingSettings(n_step=100, validation_interval=50, loss=LogSigmoidLoss(),
                                      embedding_regularisation=_zero_regulariser(),
                                      feature_regularisation=_zero_regulariser(),
                                      hidden_regularisation=_zero_regulariser(), learning_rate=0.1,
                                      learning_rate_decay=None, learning_rate_modifiers={},
                                      adam_beta_m=0.9, adam_beta_v=0.999, adam_epsilon=1e-8,
                                      weight_decay=0.0, loss_scale=None),
            execution=ExecutionSettings(device="cuda", dtype="float32", train_steps_per_program_run=5,
                                        rw_batch_size=50, predict_hr_batch_size=30,
                                        predict_tail_batch_size=50, predict_n_best=11),
            logging=LogSettings(path=None, wandb=False, steps_per_log=20, predict_at=(0.5,)),
        )

    @classmethod
    def create_wikikg90mv2(cls, n_shard: int = 8) -> "Settings":
        """The full-scale shape (91.2 M entities, 1387 relations, 768 features) on ``n_shard`` GPUs:
        TransE-L2, d=256 fp32 state with fp16 features, 512 positives and 256 shared negatives
        per shard, sampled-softmax loss."""
        s = cls.create_demo()
        s.model = dataclasses.replace(
            s.model, distance_fn="L2", n_shard=n_shard, n_entity=int(np.ceil(91230610 / n_shard) + 1),
            n_relation_type=int(n_shard * np.ceil(1387 / n_shard)), embedding_size=256,
            entity_feature_size=768, gamma=10.0)
        s.data = dataclasses.replace(s.data, dataset=WikiKg90Mv2Settings(), batch_size=512,
                                     a2a_size=768 // n_shard)
        s.training = dataclasses.replace(s.training, n_step=int(5e6), validation_interval=int(2.5e5),
                                         loss=SoftmaxLoss(correction_weight=1.0), learning_rate=1e-3,
                                         learning_rate_decay=LinearLearningRateDecay())
        s.execution = dataclasses.replace(s.execution, dtype="float32", feature_dtype="float16",
                                          train_steps_per_program_run=100, rw_batch_size=512,
                                          predict_hr_batch_size=128, predict_tail_batch_size=1024,
                                          predict_n_best=100)
        s.logging = dataclasses.replace(s.logging, steps_per_log=1000, predict_at=(0.8, 0.9))
        return s


# ---------------------------------------------------------------------------
# Batches and predictions


@dataclass
class Batch:
    """Index streams of one program run; every array is uint32 with a leading shard axis.

    remote   [n_shard, steps, batch + n_shard*a2a]  table rows to gather; unique per shard, 0 = padding
    a2a      [n_shard, steps, n_shard, a2a]         positions in ``remote`` of the rows sent to each shard
    head     [n_shard, steps, batch]                positions in ``remote`` of the head entities
    relation [n_shard, steps, batch]                relation types
    tail     [n_shard, steps, batch]                column of the true tail among the received rows
    """

    remote: np.ndarray
    a2a: np.ndarray
    head: np.ndarray
    relation: np.ndarray
    tail: np.ndarray


@dataclass
class Predictions:
    """Best candidates per query: ``shard_idx`` [..., n_best, 2] = (shard, row), ``score`` [..., n_best]."""

    shard_idx: np.ndarray
    score: np.ndarray

    def _take(self, order: np.ndarray) -> "Predictions":
        lead = self.score.shape[:-1]
        width = self.score.shape[-1]
        flat_score = self.score.reshape(-1, width)
        flat_idx = self.shard_idx.reshape(-1, width, 2)
        rows = np.arange(flat_score.shape[0])[:, None]
        k = order.shape[-1]
        return Predictions(shard_idx=flat_idx[rows, order].reshape(lead + (k, 2)),
                           score=flat_score[rows, order].reshape(lead + (k,)))

    def topk(self, k: int) -> "Predictions":
        """Keep the k highest-scoring candidates of each query (unordered)."""
        flat = self.score.reshape(-1, self.score.shape[-1])
        return self._take(np.argpartition(flat, -k, axis=1)[:, -k:])

    def sort(self) -> "Predictions":
        """Order each query's candidates by descending score."""
        flat = self.score.reshape(-1, self.score.shape[-1])
        return self._take(np.argsort(flat, axis=1)[:, ::-1])


# ---------------------------------------------------------------------------
# Engine


class Engine:
    """Owns the device state of the shards held by this process and runs the commands.

    With ``world_size == 1`` every array has the reference's leading ``[n_shard]`` axis.  With one
    process per GPU, each process passes and receives only the slices of its own shards
    (``n_shard // world_size`` consecutive shards starting at ``rank * n_shard // world_size``).
    """

    def __init__(self, settings: Settings, shard_to_entity_count: np.ndarray, rank: int = 0,
                 world_size: int = 1, exchange: Optional[Callable[[bytes], List[bytes]]] = None):
        m = settings.model
        counts = np.asarray(shard_to_entity_count)
        if counts.shape != (m.n_shard,):
            raise ValueError(f"shard_to_entity_count must have shape ({m.n_shard},)")
        if np.any(counts >= m.n_entity):
            raise ValueError("every shard must hold fewer real entities than model.n_entity rows")
        self.settings = settings
        self.shard_to_entity_count = counts
        self.rank, self.world_size = rank, world_size
        self.n_local = m.n_shard // world_size
        self.local_shards = slice(rank * self.n_local, (rank + 1) * self.n_local)
        self.random = np.random.RandomState(m.seed)

        flat = settings.engine_settings()
        if world_size > 1:
            flat["execution.rank"], flat["execution.world_size"] = rank, world_size
        module = _load_engine_module()
        self.engine = module.Engine(flat, gp_folder=str(_HERE))
        if world_size > 1:
            if exchange is None:
                raise ValueError("world_size > 1 needs an `exchange` callable (all-gather of bytes)")
            handles = exchange(self.engine.comm_export())
            self.engine.comm_connect(b"".join(handles), world_size)

        self.variable_to_shape = {name: tuple(shape) for name, shape in self.engine.run("variables", {})["variables"]}
        self.variable_to_dtype = {name: np.dtype(np.uint32 if name == "step" else np.float32)
                                  for name in self.variable_to_shape}
        self.uninitialized_variables = set(self.variable_to_shape)
        self.uninitialized_entity_data = np.ones(m.n_entity, dtype=bool)
        self.entity_data_initialized = False
        self.init_scale = m.init_scale / m.embedding_size
        self.step = 0
        self.current_learning_rate = settings.training.learning_rate
        decay = settings.training.learning_rate_decay
        self.decay_step = float(decay.step) if isinstance(decay, SteppedLearningRateDecay) else None

    # -- helpers -------------------------------------------------------------

    def _local_shape(self, shape: Sequence[int]) -> Shape:
        return (self.n_local,) + tuple(shape[1:])

    @staticmethod
    def _expect_shape(what: str, array: np.ndarray, shape: Sequence[int]) -> None:
        if tuple(array.shape) != tuple(shape):
            raise ValueError(f"'{what}' has incorrect shape, expected {tuple(shape)}, actual {array.shape}")

    @staticmethod
    def _as_engine_array(array: np.ndarray) -> np.ndarray:
        array = np.ascontiguousarray(array)
        return array.view(np.int16) if array.dtype == np.float16 else array

    def _rw_indices(self, offset: int) -> np.ndarray:
        idx = np.arange(offset, offset + self.settings.execution.rw_batch_size, dtype=np.uint32)
        idx[idx >= self.settings.model.n_entity] = 0  # overflow slots go to the padding row
        return np.ascontiguousarray(np.broadcast_to(idx, (self.n_local, idx.size)))

    def random_normal(self, shape: Shape, dtype: Union[str, np.dtype] = "float32") -> np.ndarray:
        return self.random.normal(size=shape).astype(dtype)

    def random_uniform(self, shape: Shape, low: float = 0, high: float = 1,
                       dtype: Union[str, np.dtype] = "float32") -> np.ndarray:
        return self.random.uniform(low=low, high=high, size=shape).astype(dtype)

    def random_integers(self, limit: int, shape: Shape) -> np.ndarray:
        return self.random.randint(limit, size=shape).astype(np.uint32)

    # -- variables -----------------------------------------------------------

    def write_variable(self, name: str, value_or_fn: Union[np.ndarray, Callable[[Shape], np.ndarray]]) -> None:
        shape = self.variable_to_shape[name]
        value = value_or_fn if isinstance(value_or_fn, np.ndarray) else value_or_fn(shape)
        self._expect_shape(f"write({name})", value, shape)
        self.engine.run("write", dict(name=name, value=np.ascontiguousarray(value, self.variable_to_dtype[name])))
        self.uninitialized_variables.discard(name)

    def read_variable(self, name: str) -> np.ndarray:
        dtype = self.variable_to_dtype[name]
        value = np.full(self.variable_to_shape[name], np.nan if dtype.kind == "f" else 0, dtype=dtype)
        self.engine.run("read", dict(name=name, value=value))
        return value

    def initialise_variables(self) -> None:
        """Zero the step counter and the optimiser state; draw the dense parameters."""
        s, m = self.settings, self.settings.model
        self.write_variable("step", np.zeros(m.n_shard, np.uint32))
        for name, shape in self.variable_to_shape.items():
            if name.endswith(("/adam_m", "/adam_v")):
                self.write_variable(name, np.zeros(shape, np.float32))
        rel_shape = (m.n_relation_type, s.relation_embedding_size)
        if m.score_fn == "RotatE":
            relation = self.random_uniform(rel_shape, low=-np.pi, high=np.pi)
        else:
            relation = self.random_normal(rel_shape)
        self.write_variable("relation_embedding", (self.init_scale * relation).astype(np.float32))
        if m.score_fn == "TransH":  # the hyperplane normals (src/python/poplar_kge.py:643-650)
            self.write_variable("relation_normal", (self.init_scale * self.random_normal(rel_shape)).astype(np.float32))
        prefixes = [""] if m.share_feature_networks else ["head_", "tail_"]
        for prefix in prefixes:
            w = self.random_normal((m.entity_feature_size, m.embedding_size))
            scale = self.init_scale / np.sqrt(max(1, m.entity_feature_size))
            self.write_variable(f"{prefix}feature_projection", (scale * w).astype(np.float32))
            if m.feature_mlp_size > 0 and m.entity_feature_size > 0:  # src/python/poplar_kge.py:665-688
                up = self.random_normal((2 * m.embedding_size, m.feature_mlp_size))
                self.write_variable(f"{prefix}mlp_up_projection", (self.init_scale / np.sqrt(2 * m.embedding_size) * up).astype(np.float32))
                down = self.random_normal((m.feature_mlp_size, m.embedding_size))
                self.write_variable(f"{prefix}mlp_down_projection", (self.init_scale / np.sqrt(m.feature_mlp_size) * down).astype(np.float32))

    # -- entity rows ---------------------------------------------------------

    def write_entity(self, offset: int, data: np.ndarray) -> None:
        """Initialise rows [offset, offset + rw_batch_size): fresh embedding, zero optimiser state,
        the given features ``[n_local, rw_batch_size, feature_size]``."""
        self._expect_shape("write_entity(data)", data, self._local_shape(self.settings.entity_data_w_shape))
        idx = self._rw_indices(offset)
        self.engine.run("write_entity", dict(write_indices=idx, write_features=self._as_engine_array(data)))
        self.uninitialized_entity_data[idx[0]] = False

    def write_entity_rows(self, offset: int, data: np.ndarray) -> None:
        """Write whole rows ``[n_local, rw_batch_size, 3*d + f]`` (value | adam_m | sqrt(adam_v) | feature)."""
        self._expect_shape("write_entity_rows(data)", data, self._local_shape(self.settings.entity_data_r_shape))
        idx = self._rw_indices(offset)
        self.engine.run("write_entity_rows", dict(write_indices=idx, write_data=self._as_engine_array(data)))
        self.uninitialized_entity_data[idx[0]] = False

    def read_entity(self, offset: int) -> np.ndarray:
        idx = self._rw_indices(offset)
        out = np.zeros(self._local_shape(self.settings.entity_data_r_shape), dtype=self.settings.execution.dtype)
        self.engine.run("read_entity", dict(read_indices=idx, read_data=self._as_engine_array(out)))
        return out[:, : self.settings.model.n_entity - offset]

    def _chunk_offsets(self) -> range:
        return range(0, self.settings.model.n_entity, self.settings.execution.rw_batch_size)

    def read_entity_all(self) -> np.ndarray:
        """All rows of the local shards (large models: this is the whole table in host memory)."""
        return np.concatenate([self.read_entity(o) for o in self._chunk_offsets()], axis=1)

    def _padded_chunk(self, array: np.ndarray, offset: int) -> np.ndarray:
        rw = self.settings.execution.rw_batch_size
        chunk = np.asarray(array[:, offset : offset + rw])
        if chunk.shape[1] < rw:
            chunk = np.pad(chunk, [(0, 0), (0, rw - chunk.shape[1]), (0, 0)])
        return chunk

    def initialise_all(self, entity_features: np.ndarray) -> None:
        """Reset the variables, then stream all features ``[n_local, n_entity, f]`` into the table."""
        self.initialise_variables()
        for offset in self._chunk_offsets():
            self.write_entity(offset, self._padded_chunk(entity_features, offset).astype(self.settings.execution.dtype))

    def write_all_rows(self, entity_data: np.ndarray) -> None:
        """Stream whole rows ``[n_local, n_entity, 3*d + f]`` into the table."""
        for offset in self._chunk_offsets():
            self.write_entity_rows(offset, self._padded_chunk(entity_data, offset).astype(self.settings.execution.dtype))

    def read_all(self) -> Dict[str, np.ndarray]:
        state = {name: self.read_variable(name) for name in self.variable_to_shape}
        state["entity_data"] = self.read_entity_all()
        return state

    # -- sharded checkpoints --------------------------------------------------

    DUMP_CHUNK_BYTES = 256 << 20

    def _entity_layout(self) -> Tuple[int, int, int, int]:
        layout = np.zeros(4, np.uint32)
        self.engine.run("entity_layout", dict(layout=layout))
        return tuple(int(x) for x in layout)

    def _dump_manifest(self) -> Dict[str, Any]:
        row_bytes, n_entity, _, _ = self._entity_layout()
        m, e = self.settings.model, self.settings.execution
        return dict(format=1, row_bytes=row_bytes, n_entity=n_entity, n_shard=m.n_shard, embedding_size=m.embedding_size,
                    entity_feature_size=m.entity_feature_size, score_fn=m.score_fn, dtype=str(e.dtype),
                    variables={k: list(v) for k, v in self.variable_to_shape.items()})

    def dump(self, folder: Union[str, Path]) -> None:
        """Write a checkpoint: one file per local shard holding the table exactly as it is stored
        (``entity_shard<global index>.npy``, uint32 words ``[n_entity, row_bytes / 4]``, streamed in
        chunks so that host memory holds one chunk at a time), and, from rank 0, the dense variables
        with their optimiser state and the host-side schedule (``variables.npz``, ``manifest.json``).
        With one process per GPU every process calls this with the same folder and writes only its
        own shards, so a table of any size is dumped in parallel and never gathered in one place.
        The reference offers read_entity_all / read_all, which build the whole table in host memory
        (src/python/poplar_kge.py:583-598, 707-716)."""
        folder = Path(folder)
        folder.mkdir(parents=True, exist_ok=True)
        row_bytes, n_entity, n_local, first_shard = self._entity_layout()
        words = row_bytes // 4
        chunk_rows = max(1, self.DUMP_CHUNK_BYTES // row_bytes)
        for local in range(n_local):
            out = np.lib.format.open_memmap(folder / f"entity_shard{first_shard + local:03d}.npy", mode="w+",
                                            dtype=np.uint32, shape=(n_entity, words))
            buffer = np.empty((chunk_rows, words), np.uint32)
            for first in range(0, n_entity, chunk_rows):
                count = min(chunk_rows, n_entity - first)
                self.engine.run("dump_entity_rows", dict(shard_range=np.array([local, first, count], np.uint32), rows=buffer[:count]))
                out[first : first + count] = buffer[:count]
            out.flush()
            del out
        state = {name: self.read_variable(name) for name in self.variable_to_shape}  # every process: reads may be collective
        if self.rank == 0:
            np.savez(folder / "variables.npz", **{name.replace("/", "__"): value for name, value in state.items()})
            manifest = self._dump_manifest()
            manifest["host"] = dict(step=self.step, current_learning_rate=self.current_learning_rate, decay_step=self.decay_step)
            (folder / "manifest.json").write_text(json.dumps(manifest, indent=1))

    def restore(self, folder: Union[str, Path]) -> None:
        """Load a checkpoint written by :meth:`dump` into an engine built with the same settings
        (any number of processes: each reads the files of its own shards)."""
        folder = Path(folder)
        manifest = json.loads((folder / "manifest.json").read_text())
        mine = self._dump_manifest()
        for key, value in mine.items():
            if manifest.get(key) != value:
                raise ValueError(f"checkpoint {folder} was written with {key}={manifest.get(key)!r}, this engine has {value!r}")
        row_bytes, n_entity, n_local, first_shard = self._entity_layout()
        chunk_rows = max(1, self.DUMP_CHUNK_BYTES // row_bytes)
        for local in range(n_local):
            path = folder / f"entity_shard{first_shard + local:03d}.npy"
            rows = np.load(path, mmap_mode="r")
            if rows.shape != (n_entity, row_bytes // 4) or rows.dtype != np.uint32:
                raise ValueError(f"{path} holds {rows.dtype}{rows.shape}, expected uint32{(n_entity, row_bytes // 4)}")
            for first in range(0, n_entity, chunk_rows):
                count = min(chunk_rows, n_entity - first)
                self.engine.run("restore_entity_rows", dict(shard_range=np.array([local, first, count], np.uint32),
                                                            rows=np.ascontiguousarray(rows[first : first + count])))
        with np.load(folder / "variables.npz") as state:
            for name in self.variable_to_shape:
                self.write_variable(name, state[name.replace("/", "__")])
        host = manifest["host"]
        self.step, self.current_learning_rate, self.decay_step = host["step"], host["current_learning_rate"], host["decay_step"]
        self.uninitialized_entity_data[:] = False

    # -- training ------------------------------------------------------------

    def _update_learning_rate(self) -> None:
        t, decay = self.settings.training, self.settings.training.learning_rate_decay
        if isinstance(decay, LinearLearningRateDecay):
            self.current_learning_rate = t.learning_rate * (1 - self.step / t.n_step)
        elif isinstance(decay, SteppedLearningRateDecay):
            if self.step >= self.decay_step:
                self.current_learning_rate *= decay.multiplier
                self.decay_step *= 1.5
        elif isinstance(decay, ExponentialLearningRateDecay):
            self.current_learning_rate = t.learning_rate * 0.5 ** (self.step / decay.half_life_steps)

    def train_step_loop(self, batch: Batch) -> Tuple[float, float]:
        """Run ``train_steps_per_program_run`` steps; returns (loss summed over local shards, learning rate)."""
        if not self.entity_data_initialized:
            missing = int(np.sum(self.uninitialized_entity_data))
            if missing:
                raise ValueError(f"Calling train_step() with uninitialised entity data ({missing} entities)")
            self.entity_data_initialized = True
        if self.uninitialized_variables:
            raise ValueError(f"Calling train_step() with uninitialised variables {sorted(self.uninitialized_variables)}")
        self._update_learning_rate()
        self.step += self.settings.execution.train_steps_per_program_run
        loss = np.full(self.n_local, np.nan, dtype=np.float32)
        streams = {k: np.ascontiguousarray(v, dtype=np.uint32) for k, v in vars(batch).items()}
        self.engine.run("train_step_loop", dict(
            learning_rate=np.full(self.n_local, self.current_learning_rate, dtype=np.float32), loss=loss, **streams))
        return float(np.sum(loss)), self.current_learning_rate

    # -- sampling on the device ----------------------------------------------

    @staticmethod
    def bucket_triples(train_hrt: np.ndarray, entity_to_shard: np.ndarray, entity_to_idx: np.ndarray,
                       n_shard: int) -> Dict[str, np.ndarray]:
        """The training triples as the device sampler wants them: local rows sorted by
        (head shard, tail shard) bucket with each bucket's offset and size, the index that the
        reference's ``Dataset`` builds for ``sample_batch`` (src/python/poplar_kge_dataset.py:199-241)."""
        hrt = np.asarray(train_hrt)
        head_shard, tail_shard = entity_to_shard[hrt[:, 0]], entity_to_shard[hrt[:, 2]]
        pair = n_shard * head_shard.astype(np.int64) + tail_shard
        order = np.argsort(pair, kind="stable")
        count = np.bincount(pair, minlength=n_shard * n_shard)
        offset = np.concatenate([[0], np.cumsum(count)[:-1]])
        ordered = hrt[order]
        triples = np.stack([entity_to_idx[ordered[:, 0]], ordered[:, 1], entity_to_idx[ordered[:, 2]]]).astype(np.uint32)
        return dict(triples=np.ascontiguousarray(triples), bucket_offset=offset.reshape(n_shard, n_shard).astype(np.uint32),
                    bucket_count=count.reshape(n_shard, n_shard).astype(np.uint32))

    def load_triples(self, train_hrt: np.ndarray, entity_to_shard: np.ndarray, entity_to_idx: np.ndarray) -> None:
        """Put the training set on the device for ``sample_batch`` / ``train_step_loop_sampled``."""
        n = self.settings.model.n_shard
        self.engine.run("load_triples", dict(
            shard_to_count=np.ascontiguousarray(self.shard_to_entity_count, dtype=np.uint32),
            **self.bucket_triples(train_hrt, np.asarray(entity_to_shard), np.asarray(entity_to_idx), n)))

    def sample_batch(self, seed: int) -> Batch:
        """One program run's index streams of the local shards, drawn on the device (and left staged
        there): the device counterpart of ``Dataset.sample_batch`` (src/python/poplar_kge_dataset.py:310-393)."""
        d, e, n = self.settings.data, self.settings.execution, self.settings.model.n_shard
        S, B, R = e.train_steps_per_program_run, d.batch_size, d.batch_size + n * d.a2a_size
        out = dict(remote=np.zeros((self.n_local, S, R), np.uint32), a2a=np.zeros((self.n_local, S, n, d.a2a_size), np.uint32),
                   head=np.zeros((self.n_local, S, B), np.uint32), relation=np.zeros((self.n_local, S, B), np.uint32),
                   tail=np.zeros((self.n_local, S, B), np.uint32))
        self.engine.run("sample_batch", dict(sample_seed=np.array([seed], np.uint32), **out))
        return Batch(**out)

    def train_step_loop_sampled(self, seed: int) -> Tuple[float, float]:
        """``train_step_loop`` on a batch that the device draws itself: no index array crosses the host."""
        if self.uninitialized_variables:
            raise ValueError(f"Calling train_step() with uninitialised variables {sorted(self.uninitialized_variables)}")
        self._update_learning_rate()
        self.step += self.settings.execution.train_steps_per_program_run
        loss = np.full(self.n_local, np.nan, dtype=np.float32)
        self.engine.run("train_step_loop_sampled", dict(
            sample_seed=np.array([seed], np.uint32), loss=loss,
            learning_rate=np.full(self.n_local, self.current_learning_rate, dtype=np.float32)))
        return float(np.sum(loss)), self.current_learning_rate

    # -- prediction ----------------------------------------------------------

    def _predict_hr_chunk(self, idx_relation: np.ndarray) -> Predictions:
        e, n = self.settings.execution, self.settings.model.n_shard
        scores = np.full((self.n_local, n, e.predict_hr_batch_size, e.predict_n_best), np.nan, dtype=np.float32)
        indices = np.zeros(scores.shape, dtype=np.uint32)
        self.engine.run("predict", dict(
            predict_head=np.ascontiguousarray(idx_relation[:, :, 0], dtype=np.uint32),
            predict_relation=np.ascontiguousarray(idx_relation[:, :, 1], dtype=np.uint32),
            predict_entity_count=np.ascontiguousarray(self.shard_to_entity_count[self.local_shards], dtype=np.uint32),
            predict_scores=scores, predict_indices=indices))
        shard_idx = np.empty(indices.shape + (2,), dtype=np.uint32)
        shard_idx[..., 0] = np.arange(n, dtype=np.uint32)[None, :, None, None]
        shard_idx[..., 1] = indices
        merged = Predictions(
            shard_idx=shard_idx.transpose(0, 2, 1, 3, 4).reshape(self.n_local, e.predict_hr_batch_size, -1, 2),
            score=scores.transpose(0, 2, 1, 3).reshape(self.n_local, e.predict_hr_batch_size, -1))
        return merged.topk(e.predict_n_best).sort()

    def predict_chunks(self, query_shards: np.ndarray) -> int:
        """Engine "predict" calls needed for queries whose head shards are ``query_shards``: the
        same on every process, whatever shards it holds."""
        counts = np.bincount(np.asarray(query_shards, np.int64), minlength=self.settings.model.n_shard)
        hr = self.settings.execution.predict_hr_batch_size
        return int(-(-int(counts.max(initial=0)) // hr))

    def predict(self, shard_idx_relation: np.ndarray) -> Predictions:
        """Rank all entities as tails of (head shard, head row, relation) queries ``[q, 3]``.

        Queries whose head lives on a shard of another process are left as zeros.  With
        world_size > 1 every process passes the same query list: the number of engine calls is taken
        from the longest per-shard list over ALL shards, so that every process makes the same number
        of calls (each engine call synchronises the processes twice), padding with empty chunks."""
        q = np.asarray(shard_idx_relation)
        if q.ndim != 2 or q.shape[1] != 3:
            raise ValueError("shard_idx_relation should be of shape (n, 3)")
        e = self.settings.execution
        local = list(range(self.local_shards.start, self.local_shards.stop))
        per_shard = [np.flatnonzero(q[:, 0] == s) for s in local]
        out = Predictions(shard_idx=np.zeros((q.shape[0], e.predict_n_best, 2), np.uint32),
                          score=np.zeros((q.shape[0], e.predict_n_best), np.float32))
        for lo in range(0, self.predict_chunks(q[:, 0]) * e.predict_hr_batch_size, e.predict_hr_batch_size):
            chunk = np.zeros((self.n_local, e.predict_hr_batch_size, 2), dtype=np.uint32)
            picks = [x[lo : lo + e.predict_hr_batch_size] for x in per_shard]
            for l, rows in enumerate(picks):
                chunk[l, : len(rows)] = q[rows, 1:3]
            result = self._predict_hr_chunk(chunk)
            for l, rows in enumerate(picks):
                out.shard_idx[rows] = result.shard_idx[l, : len(rows)]
                out.score[rows] = result.score[l, : len(rows)]
        return out
