"""numpy restatement of the reference's sharded KGE training step and predict.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).  Every function names the
reference lines it restates; paths are relative to the reference project root.

All shards are evaluated in one process with a leading ``[n_shard]`` axis, which
is exactly how the reference presents them to its host API
(src/poplar_kge.cpp:874-877).  The compute dtype is a parameter: ``float64`` is
the ground truth the CUDA path is compared with, ``float32`` reproduces the
reference's arithmetic width.
"""

from __future__ import annotations

import dataclasses
from typing import Dict, Optional, Tuple

import numpy as np

# ---------------------------------------------------------------------------
# Configuration (the keys the engine reads: src/poplar_kge.cpp:198-246)


@dataclasses.dataclass
class StepConfig:
    n_shard: int
    n_entity: int  # rows per shard, including the padding row 0
    n_relation_type: int
    embedding_size: int
    entity_feature_size: int
    batch_size: int  # positives per shard
    a2a_size: int  # tails sent to each peer
    score_fn: str = "TransE"  # TransE | DistMult | ComplEx | RotatE
    distance_fn: str = "L1"  # L1 | L2 | MatMul
    gamma: float = 10.0
    loss_type: str = "logsigmoid"  # logsigmoid | softmax
    correction_weight: float = 0.0
    negative_adversarial_scale: float = 0.0
    share_feature_networks: bool = True
    adam_beta_m: float = 0.9
    adam_beta_v: float = 0.999
    adam_epsilon: float = 1e-8
    weight_decay: float = 0.0
    loss_scale: Optional[float] = None
    learning_rate_modifiers: Dict[str, float] = dataclasses.field(default_factory=dict)
    # (power, weight) of the norm regularisers (src/poplar_kge.cpp:144-152, 175-177)
    embedding_regularisation: Tuple[float, float] = (2.0, 0.0)
    feature_regularisation: Tuple[float, float] = (2.0, 0.0)
    hidden_regularisation: Tuple[float, float] = (2.0, 0.0)
    feature_dropout: float = 0.0  # src/poplar_kge.cpp:459-461
    feature_mlp_size: int = 0  # src/poplar_kge.cpp:453-458

    def __post_init__(self) -> None:
        if self.loss_scale is None:
            # src/python/poplar_kge.py:259-262
            self.loss_scale = float(self.batch_size * self.n_shard * self.a2a_size)

    @property
    def n_tail(self) -> int:  # src/python/poplar_kge.py:197-199
        return self.n_shard * self.a2a_size

    @property
    def n_remote(self) -> int:  # src/python/poplar_kge.py:201-203
        return self.batch_size + self.n_tail

    @property
    def row_size(self) -> int:  # src/poplar_kge.cpp:274-275
        return 3 * self.embedding_size + self.entity_feature_size

    @property
    def projection_names(self) -> Tuple[str, ...]:  # src/poplar_kge.cpp:268-273
        if self.share_feature_networks:
            return ("feature_projection",)
        return ("head_feature_projection", "tail_feature_projection")


# ---------------------------------------------------------------------------
# Elementary ops, each with the backward the reference's tape would replay


def l1_distance(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """out[i, j] = sum_k abs(a[i, k] - b[j, k]).

    src/poplar_extensions/l1distance.codelet.cpp:49-56 (portable ``l1dist``).
    """
    out = np.empty((a.shape[0], b.shape[0]), dtype=a.dtype)
    for lo in range(0, a.shape[0], 64):
        out[lo : lo + 64] = np.abs(a[lo : lo + 64, None, :] - b[None, :, :]).sum(-1)
    return out


def l1_distance_grad(a: np.ndarray, b: np.ndarray, grad_out: np.ndarray) -> np.ndarray:
    """grad_a[i, k] = sum_j grad_out[i, j] * sign(a[i, k] - b[j, k]), sign(0) = 0.

    src/poplar_extensions/l1distance.codelet.cpp:76-79,138-145 (``signum``,
    ``l1distgrad``).  The gradient for ``b`` is the same function with the
    arguments swapped and ``grad_out`` transposed (src/pag/pag.cpp:791-803).
    """
    out = np.empty_like(a)
    for lo in range(0, a.shape[0], 64):
        sgn = np.sign(a[lo : lo + 64, None, :] - b[None, :, :])
        out[lo : lo + 64] = np.einsum("ij,ijk->ik", grad_out[lo : lo + 64], sgn)
    return out


def l2_distance(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """out[i, j] = sqrt(sum_k (a[i, k] - b[j, k])^2): a true Euclidean distance.

    src/poplar_extensions/l2distance.codelet.cpp:54-62 (portable ``l2dist``).
    """
    out = np.empty((a.shape[0], b.shape[0]), dtype=a.dtype)
    for lo in range(0, a.shape[0], 64):
        diff = a[lo : lo + 64, None, :] - b[None, :, :]
        out[lo : lo + 64] = np.sqrt((diff * diff).sum(-1))
    return out


def l2_distance_grad(
    a: np.ndarray, b: np.ndarray, dist: np.ndarray, grad_out: np.ndarray
) -> np.ndarray:
    """grad_a[i, k] = sum_j grad_out[i, j] * (a[i, k] - b[j, k]) / dist[i, j], 0 where dist is 0.

    src/poplar_extensions/l2distance.codelet.cpp:149-158 (portable ``l2distgrad``).
    """
    with np.errstate(divide="ignore", invalid="ignore"):
        coeff = np.where(dist == 0, 0, grad_out / np.where(dist == 0, 1, dist))
    out = np.empty_like(a)
    for lo in range(0, a.shape[0], 64):
        diff = a[lo : lo + 64, None, :] - b[None, :, :]
        out[lo : lo + 64] = np.einsum("ij,ijk->ik", coeff[lo : lo + 64], diff)
    return out


def log_sigmoid(x: np.ndarray) -> np.ndarray:
    """Guarded log-sigmoid: ``x`` itself at or below -11, else -log1p(exp(-x)).

    src/pag/pag.cpp:893-896.
    """
    return np.where(x > -11, -np.log1p(np.exp(-np.maximum(x, -11))), x)


def log_sigmoid_grad(x: np.ndarray, grad_out: np.ndarray) -> np.ndarray:
    """grad_out / (1 + exp(min(x, 11))).  src/pag/pag.cpp:901-904."""
    return grad_out / (1 + np.exp(np.minimum(x, 11)))


def log_softmax(x: np.ndarray) -> np.ndarray:
    """Row-wise stable log-softmax (popnn::logSoftmax, src/pag/pag.cpp:846-848)."""
    shifted = x - x.max(axis=-1, keepdims=True)
    return shifted - np.log(np.exp(shifted).sum(axis=-1, keepdims=True))


def log_softmax_grad(logp: np.ndarray, grad_out: np.ndarray) -> np.ndarray:
    """grad_out - sum(grad_out) * exp(logp).  src/pag/pag.cpp:851-860."""
    return grad_out - grad_out.sum(axis=-1, keepdims=True) * np.exp(logp)


def scatter_add_rows(n_rows: int, indices: np.ndarray, rows: np.ndarray) -> np.ndarray:
    """Dense zero table with ``rows`` added at ``indices`` (duplicates accumulate).

    The backward of a row gather: src/pag/pag.cpp:721-743 (``multiUpdateAdd``).
    """
    out = np.zeros((n_rows,) + rows.shape[1:], dtype=rows.dtype)
    np.add.at(out, indices, rows)
    return out


def lp_norm(a: np.ndarray, p: float) -> np.ndarray:
    """Rows' (sum_k |a_k^p|)^(1/p) (lpnorm, src/poplar_kge.cpp:389-391).  |a|^p stands for |a^p|:
    the same wherever a^p is defined (integer p, or a >= 0)."""
    return np.sum(np.abs(a) ** p, axis=-1) ** (1.0 / p)


def lp_norm_grad(a: np.ndarray, p: float, grad_out: np.ndarray) -> np.ndarray:
    """Backward of lp_norm as the reference's tape replays it: pow gives g * exponent * out / base
    with 0 where the base is 0 (src/pag/pag.cpp:493-503), abs gives sign(x) * g (:449-456), the
    sum broadcasts."""
    u = np.abs(a) ** p
    s = np.sum(u, axis=-1, keepdims=True)
    norm = s ** (1.0 / p)
    d_s = grad_out[..., None] * (1.0 / p) * norm / (s + (s == 0))  # outer pow
    return d_s * p * u / (a + (a == 0))  # abs, then the inner pow: sign(a^p) * p * a^p / a


def all_to_all(blocks: np.ndarray) -> np.ndarray:
    """out[dst, src] = blocks[src, dst] on the stacked shard axis.

    src/pag/pag.cpp:915-935; the backward is the same exchange applied to the
    gradient (:925-932).
    """
    return np.swapaxes(blocks, 0, 1)


def _f32(x) -> np.float32:
    """The engine holds its hyper-parameters as C++ ``float`` (src/poplar_kge.cpp:167-179, 213-216),
    so constants derived from them, like 1 - beta, are float32 arithmetic on float32 values."""
    return np.float32(x)


def adam_step_size(step: int, lr, beta_m: float, beta_v: float, dtype) -> np.ndarray:
    """lr * sqrt(1 - beta_v^t) / (1 - beta_m^t) with ``t`` already incremented.

    src/fructose/frnn.cpp:42-59.
    """
    t = dtype(step)
    return (np.sqrt(1 - dtype(_f32(beta_v)) ** t) / (1 - dtype(_f32(beta_m)) ** t)) * dtype(_f32(lr))


def adam_update(x, m, v, grad, step_size, cfg: StepConfig):
    """In-place Adam in the reference's form (epsilon outside the bias correction,
    decoupled weight decay).  src/fructose/frnn.cpp:61-90.
    """
    dt = x.dtype.type
    beta_m, beta_v = _f32(cfg.adam_beta_m), _f32(cfg.adam_beta_v)
    m *= dt(beta_m)
    m += dt(_f32(1) - beta_m) * grad
    v *= dt(beta_v)
    v += dt(_f32(1) - beta_v) * grad * grad
    x -= step_size * (m / (np.sqrt(v) + dt(_f32(cfg.adam_epsilon))) + dt(_f32(cfg.weight_decay)) * x)


# ---------------------------------------------------------------------------
# Score functions (src/poplar_kge.cpp:488-613)


def predict_tail(cfg: StepConfig, h: np.ndarray, r: np.ndarray) -> np.ndarray:
    if cfg.score_fn == "TransE":  # :488-490
        return h + r
    if cfg.score_fn == "DistMult":  # :567-569
        return h * r
    if cfg.score_fn == "ComplEx":  # :501-510 (first half real, second half imaginary)
        half = h.shape[-1] // 2
        hr, hi, rr, ri = h[..., :half], h[..., half:], r[..., :half], r[..., half:]
        return np.concatenate([hr * rr - hi * ri, hr * ri + hi * rr], axis=-1)
    if cfg.score_fn == "RotatE":  # :516-530: the angles go through float16, and so do their sine and cosine
        half = h.shape[-1] // 2
        re, im = h[..., :half], h[..., half:]
        sin, cos = _rotate_sin_cos(r, h.dtype)
        return np.concatenate([re * cos - im * sin, im * cos + re * sin], axis=-1)
    if cfg.score_fn == "TransH":  # :539-550: r = relation row | normal row; returns unit normal | predicted tail
        d = h.shape[-1]
        rel, w = r[..., :d], r[..., d:]
        n = w / np.sqrt(np.sum(w * w, axis=-1, keepdims=True))
        projected = h - n * np.sum(n * h, axis=-1, keepdims=True)
        return np.concatenate([n, projected + rel], axis=-1)
    raise ValueError(f"score_fn {cfg.score_fn!r} is not covered by the oracle")


def _rotate_sin_cos(r: np.ndarray, dtype) -> Tuple[np.ndarray, np.ndarray]:
    """sin and cos of the relation angles as src/poplar_kge.cpp:522-525 computes them: the angles are
    cast to float16, sine and cosine are taken in float16 (restated as the correctly rounded
    float16 of the exact value), and the results are cast back."""
    theta = r.astype(np.float16).astype(np.float64)
    return np.sin(theta).astype(np.float16).astype(dtype), np.cos(theta).astype(np.float16).astype(dtype)


def predict_tail_grad(cfg: StepConfig, h, r, dp) -> Tuple[np.ndarray, np.ndarray]:
    if cfg.score_fn == "TransE":
        return dp, dp
    if cfg.score_fn == "DistMult":
        return dp * r, dp * h
    if cfg.score_fn == "ComplEx":
        half = h.shape[-1] // 2
        hr, hi, rr, ri = h[..., :half], h[..., half:], r[..., :half], r[..., half:]
        dpr, dpi = dp[..., :half], dp[..., half:]
        dh = np.concatenate([dpr * rr + dpi * ri, -dpr * ri + dpi * rr], axis=-1)
        dr = np.concatenate([dpr * hr + dpi * hi, -dpr * hi + dpi * hr], axis=-1)
        return dh, dr
    if cfg.score_fn == "RotatE":
        # The gradients of sine and cosine pass through the float16 casts (src/pag/pag.cpp:619-633:
        # the gradient of a cast is cast to the input's type), and the backward of sin / cos runs in
        # float16 (:552-595: grad * cos(x), -grad * sin(x) on the float16 tensor); the two are added
        # in float16 and cast back to float32 for the relation table.
        half = h.shape[-1] // 2
        re, im = h[..., :half], h[..., half:]
        sin, cos = _rotate_sin_cos(r, h.dtype)
        dpr, dpi = dp[..., :half], dp[..., half:]
        dh = np.concatenate([dpr * cos + dpi * sin, -dpr * sin + dpi * cos], axis=-1)
        d_sin = (-dpr * im + dpi * re).astype(np.float16)
        d_cos = (dpr * re + dpi * im).astype(np.float16)
        f16 = lambda x: x.astype(np.float16)  # noqa: E731
        via_sin = f16(d_sin.astype(np.float64) * f16(cos).astype(np.float64))
        via_cos = f16(-d_cos.astype(np.float64) * f16(sin).astype(np.float64))
        d_theta = f16(via_sin.astype(np.float64) + via_cos.astype(np.float64)).astype(h.dtype)
        return dh, d_theta
    if cfg.score_fn == "TransH":  # backward of :539-550; dp = d unit normal | d predicted tail
        d = h.shape[-1]
        w = r[..., d:]
        norm = np.sqrt(np.sum(w * w, axis=-1, keepdims=True))
        n = w / norm
        d_n, d_pt = dp[..., :d], dp[..., d:]
        a = np.sum(n * h, axis=-1, keepdims=True)
        b = np.sum(n * d_pt, axis=-1, keepdims=True)
        d_h = d_pt - n * b
        d_n = d_n - a * d_pt - h * b
        d_w = (d_n - n * np.sum(n * d_n, axis=-1, keepdims=True)) / norm  # through w / |w|
        return d_h, np.concatenate([d_pt, d_w], axis=-1)
    raise ValueError(cfg.score_fn)


def transh_distance(p: np.ndarray, tails: np.ndarray):
    """sum_k |pt_ik - (t_jk - n_ik (n_i . t_j))| (src/poplar_kge.cpp:552-565) for p = unit normal |
    predicted tail; also the per-pair element differences' signs and the projections n_i . t_j."""
    d = tails.shape[-1]
    n, pt = p[..., :d], p[..., d:]
    s = n @ tails.T  # [B, T]
    e = pt[:, None, :] - tails[None, :, :] + n[:, None, :] * s[:, :, None]
    return np.sum(np.abs(e), axis=-1), np.sign(e), s


def transh_distance_grad(p: np.ndarray, tails: np.ndarray, g: np.ndarray):
    """Gradients of transh_distance times g [B, T] with respect to p [B, 2D] and tails [T, D]."""
    d = tails.shape[-1]
    n = p[..., :d]
    _, sg, s = transh_distance(p, tails)
    u = np.einsum("ijk,ik->ij", sg, n)  # the signs' sum along the normal
    d_pt = np.einsum("ij,ijk->ik", g, sg)
    d_n = np.einsum("ij,ijk->ik", g * s, sg) + (g * u) @ tails
    d_t = -np.einsum("ij,ijk->jk", g, sg) + (g * u).T @ n
    return np.concatenate([d_n, d_pt], axis=-1), d_t


def _distance(cfg: StepConfig, a, b):  # src/poplar_kge.cpp:469-486
    if cfg.distance_fn in ("L1", "L1_old"):
        return l1_distance(a, b)
    if cfg.distance_fn in ("L2", "L2_old"):
        return l2_distance(a, b)
    if cfg.distance_fn == "MatMul":
        return a @ b.T
    raise ValueError(f"distance_fn {cfg.distance_fn!r}")


def _distance_grad(cfg: StepConfig, a, b, dist, g):
    if cfg.distance_fn in ("L1", "L1_old"):
        return l1_distance_grad(a, b, g), l1_distance_grad(b, a, g.T)
    if cfg.distance_fn in ("L2", "L2_old"):
        return l2_distance_grad(a, b, dist, g), l2_distance_grad(b, a, dist.T, g.T)
    return g @ b, g.T @ a  # src/pag/pag.cpp:685-701


def score(cfg: StepConfig, p: np.ndarray, tails: np.ndarray):
    """Scores [B, T] and the raw distance the backward needs.

    TransE: gamma - distance (:492-499).  DistMult / ComplEx: distance(p, tails)
    as is (:512-514, :571-573), normally with distance_fn "MatMul".
    """
    if cfg.score_fn == "TransH":  # :552-565, whatever distance_fn says
        dist = transh_distance(p, tails)[0]
        return p.dtype.type(_f32(cfg.gamma)) - dist, dist
    dist = _distance(cfg, p, tails)
    if cfg.score_fn in ("TransE", "RotatE"):  # :492-499, :532-537
        return p.dtype.type(_f32(cfg.gamma)) - dist, dist
    return dist, dist


def score_grad(cfg: StepConfig, p, tails, dist, g):
    if cfg.score_fn == "TransH":
        return transh_distance_grad(p, tails, -g)
    if cfg.score_fn in ("TransE", "RotatE"):
        g = -g
    return _distance_grad(cfg, p, tails, dist, g)


# ---------------------------------------------------------------------------
# Losses (src/poplar_kge.cpp:615-660).  Each returns (loss, dloss/dscores).


def loss_logsigmoid(cfg: StepConfig, scores: np.ndarray, labels: np.ndarray):
    dt = scores.dtype.type
    n_tail = cfg.n_tail
    onehot = np.zeros_like(scores)
    onehot[np.arange(scores.shape[0]), labels] = 1
    w_neg = dt(_f32(0.5 * n_tail) / _f32(n_tail - 1))  # float arithmetic in the reference (:619-620)
    w_pos = dt(_f32(0.5 * n_tail))
    weight = (w_pos - w_neg) * onehot + w_neg
    if cfg.negative_adversarial_scale > 0:  # :623-633, softmax is detached
        z = dt(_f32(cfg.negative_adversarial_scale)) * scores + dt(-10000.0) * onehot
        z = z - z.max(axis=-1, keepdims=True)
        soft = np.exp(z)
        soft /= soft.sum(axis=-1, keepdims=True)
        weight = weight * (onehot + dt(n_tail - 1) * soft)
    mask = 2 * onehot - 1
    denom = dt(cfg.n_shard * cfg.batch_size * cfg.a2a_size * cfg.n_shard)
    x = mask * scores
    loss = -(weight * log_sigmoid(x)).sum() / denom
    dscores = mask * log_sigmoid_grad(x, -weight / denom)
    return loss, dscores


def softmax_correction(cfg: StepConfig) -> float:
    """log(n_entity * n_shard - 1) - log(n_shard * a2a - 1), rounded to float32 (:644)."""
    return float(
        np.float32(
            np.log(float(cfg.n_entity * cfg.n_shard - 1)) - np.log(float(cfg.n_tail - 1))
        )
    )


def loss_softmax(cfg: StepConfig, scores: np.ndarray, labels: np.ndarray):
    dt = scores.dtype.type
    onehot = np.zeros_like(scores)
    onehot[np.arange(scores.shape[0]), labels] = 1
    corrected = scores
    if cfg.correction_weight:
        shift = dt(np.float32(cfg.correction_weight) * np.float32(softmax_correction(cfg)))
        corrected = scores + shift * (1 - onehot)
    logp = log_softmax(corrected)
    denom = dt(cfg.n_shard * cfg.batch_size)
    loss = -(logp * onehot).sum() / denom  # src/fructose/frnn.cpp:18-23
    dscores = log_softmax_grad(logp, -onehot / denom)
    return loss, dscores


def loss_and_grad(cfg: StepConfig, scores, labels):
    if cfg.loss_type == "logsigmoid":
        return loss_logsigmoid(cfg, scores, labels)
    if cfg.loss_type == "softmax":
        return loss_softmax(cfg, scores, labels)
    raise ValueError(f"loss type {cfg.loss_type!r}")


# ---------------------------------------------------------------------------
# The model state and the step


class Oracle:
    """State + ``train_step`` / ``train_step_loop`` / ``predict``.

    ``entity_data`` is the stacked table ``[n_shard, n_entity, 3D+F]`` with row
    layout value | adam_m | sqrt(adam_v) | feature (src/poplar_kge.cpp:405-417).
    Dense parameters are held once (they are replicated across shards in effect:
    slices are all-gathered on every use and gradients reduce-scattered,
    src/poplar_kge.cpp:341-348, src/pag/pag.cpp:980-994).
    """

    def __init__(self, cfg: StepConfig, dtype=np.float64):
        self.cfg = cfg
        self.dtype = np.dtype(dtype).type
        d, f = cfg.embedding_size, cfg.entity_feature_size
        self.entity_data = np.zeros((cfg.n_shard, cfg.n_entity, cfg.row_size), dtype)
        self.variables: Dict[str, np.ndarray] = {}
        # RotatE's relations are angles, one per complex pair (src/poplar_kge.cpp:248-251)
        shapes = {"relation_embedding": (cfg.n_relation_type, d // 2 if cfg.score_fn == "RotatE" else d)}
        if cfg.score_fn == "TransH":  # src/poplar_kge.cpp:252-255
            shapes["relation_normal"] = (cfg.n_relation_type, d)
        for name in cfg.projection_names:
            shapes[name] = (f, d)
            if cfg.feature_mlp_size > 0:  # src/poplar_kge.cpp:260-265
                prefix = name[: -len("feature_projection")]
                shapes[prefix + "mlp_up_projection"] = (2 * d, cfg.feature_mlp_size)
                shapes[prefix + "mlp_down_projection"] = (cfg.feature_mlp_size, d)
        for name, shape in shapes.items():
            for suffix in ("", "/adam_m", "/adam_v"):
                self.variables[name + suffix] = np.zeros(shape, dtype)
        self.step = 0
        self.dropout_mask = None  # callable (training step number, call 0 head / 1 tail) -> bool [n_shard, R, D]
        self.last = {}  # intermediates of the most recent step, for kernel-level checks

    # -- state I/O ---------------------------------------------------------

    def set_state(self, state: Dict[str, np.ndarray]) -> None:
        for key, value in state.items():
            if key == "entity_data":
                self.entity_data[...] = value
            elif key == "step":
                (self.step,) = {int(s) for s in np.atleast_1d(value)}
            else:
                self.variables[key][...] = value

    def get_state(self) -> Dict[str, np.ndarray]:
        out = {k: v.copy() for k, v in self.variables.items()}
        out["entity_data"] = self.entity_data.copy()
        out["step"] = np.full(self.cfg.n_shard, self.step, np.uint32)
        return out

    # -- training ----------------------------------------------------------

    def _relation_rows(self) -> np.ndarray:
        """The rows predict_tail gathers: the relation embedding, for TransH followed by the normal."""
        rel = self.variables["relation_embedding"]
        if self.cfg.score_fn == "TransH":
            return np.concatenate([rel, self.variables["relation_normal"]], axis=-1)
        return rel

    def _mlp(self, part: str, kind: str) -> str:
        prefix = "" if self.cfg.share_feature_networks else f"{part}_"
        return f"{prefix}mlp_{kind}_projection"

    def _projection(self, part: str) -> str:
        if self.cfg.share_feature_networks:
            return "feature_projection"
        return f"{part}_feature_projection"

    def train_step(self, lr: float, remote, a2a, head, relation, tail) -> np.ndarray:
        """One step of src/poplar_kge.cpp:664-707 for every shard; returns loss[n_shard]."""
        cfg, dt = self.cfg, self.dtype
        n, d = cfg.n_shard, cfg.embedding_size
        remote, a2a, head, relation, tail = (
            np.asarray(x).astype(np.int64) for x in (remote, a2a, head, relation, tail)
        )
        rel = self._relation_rows()
        w_head = self.variables[self._projection("head")]
        w_tail = self.variables[self._projection("tail")]

        # 1. gather rows (:671, :405-410)
        rows = np.stack([self.entity_data[s, remote[s]] for s in range(n)])
        value, adam_m, sqrt_v, feat = (
            rows[..., :d],
            rows[..., d : 2 * d].copy(),
            rows[..., 2 * d : 3 * d],
            rows[..., 3 * d :],
        )
        value = value.copy()
        # 2. hidden, lookups, exchange (:676-681, :439-467)
        mlp = []  # per call: (concatenated input, pre-activation, up projection, down projection)
        fh_h, fh_t = feat @ w_head, feat @ w_tail
        if cfg.feature_mlp_size > 0:
            # :453-458: featureHidden = relu(concat(value, featureHidden) . up) . down
            outs = []
            for part, fh0 in (("head", fh_h), ("tail", fh_t)):
                up, down = self.variables[self._mlp(part, "up")], self.variables[self._mlp(part, "down")]
                cat = np.concatenate([value, fh0], axis=-1)
                pre = cat @ up
                outs.append(np.maximum(pre, 0) @ down)
                mlp.append((cat, pre, up, down))
            fh_h, fh_t = outs
        keep_h = keep_t = None
        if cfg.feature_dropout > 0 and cfg.entity_feature_size > 0:
            # frnn::dropout (src/pag/pag.cpp:596-617): kept with probability 1 - p, scaled by 1 / (1 - p);
            # each entityHidden call draws its own mask.  The masks come from `dropout_mask(step, part)`
            # -> bool [n_shard, R, D] (the reference draws them from the IPU's generator).
            scale = dt(1.0) / (dt(1.0) - dt(_f32(cfg.feature_dropout)))
            keep_h = self.dropout_mask(self.step + 1, 0) * scale
            keep_t = self.dropout_mask(self.step + 1, 1) * scale
            fh_h, fh_t = fh_h * keep_h, fh_t * keep_t
        hid_h = value + fh_h
        hid_t = hid_h if cfg.share_feature_networks and keep_h is None else value + fh_t
        heads = np.stack([hid_h[s, head[s]] for s in range(n)])
        send = np.stack([hid_t[s, a2a[s]] for s in range(n)])  # [src, dst, a2a, D]
        tails = all_to_all(send).reshape(n, cfg.n_tail, d)  # [dst, src*a2a, D]
        # norm regularisers: every entityHidden call (head part, tail part) adds its three terms to
        # the shard's loss, not normalised (:430-437, 463-465, 673-688); root gradient loss_scale (:691)
        reg_loss = np.zeros(n, self.entity_data.dtype)
        reg_value = np.zeros_like(value)                      # gradient of the gathered values
        reg_fh = [np.zeros_like(value), np.zeros_like(value)]  # gradient of each call's feature-network output
        ls = dt(_f32(cfg.loss_scale))
        for call, (hid, fh) in enumerate(((hid_h, fh_h), (hid_t, fh_t))):
            terms = ((cfg.embedding_regularisation, value, "value"), (cfg.feature_regularisation, fh, "fh"),
                     (cfg.hidden_regularisation, hid, "hidden"))
            for (power, weight), tensor, kind in terms:
                if weight <= 0:
                    continue
                wt = dt(_f32(weight))
                reg_loss += wt * np.sum(lp_norm(tensor, power), axis=-1)
                g = lp_norm_grad(tensor, power, np.full(tensor.shape[:-1], wt * ls, tensor.dtype))
                if kind in ("value", "hidden"):
                    reg_value += g
                if kind in ("fh", "hidden"):
                    reg_fh[call] += g
        # 3./4. scores and loss (:684-688)
        losses = np.zeros(n, self.entity_data.dtype)
        d_hid_h = np.zeros_like(hid_h)
        d_tails = np.zeros_like(tails)
        d_rel = np.zeros_like(rel)
        keep = {"hidden": hid_h, "tails": tails, "scores": [], "dscores": [], "pred": []}
        for s in range(n):
            r = rel[relation[s]]
            pred = predict_tail(cfg, heads[s], r)
            scores, dist = score(cfg, pred, tails[s])
            losses[s], dscores = loss_and_grad(cfg, scores, tail[s])
            dscores = dscores * dt(_f32(cfg.loss_scale))  # root gradient, never unscaled (:691)
            d_pred, d_tails[s] = score_grad(cfg, pred, tails[s], dist, dscores)
            d_head, d_r = predict_tail_grad(cfg, heads[s], r, d_pred)
            d_rel += scatter_add_rows(rel.shape[0], relation[s], d_r)
            d_hid_h[s] = scatter_add_rows(cfg.n_remote, head[s], d_head)
            keep["scores"].append(scores)
            keep["dscores"].append(dscores)
            keep["pred"].append(pred)
        # 5. exchange backward, lookups backward, projection backward
        d_send = all_to_all(d_tails.reshape(n, n, cfg.a2a_size, d))  # [src, dst, a2a, D]
        d_hid_t = np.stack(
            [
                scatter_add_rows(cfg.n_remote, a2a[s].reshape(-1), d_send[s].reshape(-1, d))
                for s in range(n)
            ]
        )
        d_value = d_hid_h + d_hid_t + reg_value
        d_fh_h, d_fh_t = d_hid_h + reg_fh[0], d_hid_t + reg_fh[1]
        if keep_h is not None:  # backward of the dropout: g / (1 - p) where the output is not zero
            d_fh_h, d_fh_t = d_fh_h * keep_h * (fh_h != 0), d_fh_t * keep_t * (fh_t != 0)
        losses = losses + reg_loss
        grads = {"relation_embedding": d_rel}
        if cfg.score_fn == "TransH":
            grads = {"relation_embedding": d_rel[:, :d], "relation_normal": d_rel[:, d:]}
        keep["d_mlp_output"] = d_fh_h + d_fh_t if cfg.share_feature_networks else d_fh_h
        if mlp:
            # backward of the MLP; max(x, 0) passes the gradient where x equals the output, zero included
            # (src/pag/pag.cpp:650-658)
            back = []
            for part, d_out, (cat, pre, up, down) in (("head", d_fh_h, mlp[0]), ("tail", d_fh_t, mlp[1])):
                boom = np.maximum(pre, 0)
                d_pre = (d_out @ down.T) * (pre == boom)
                for kind, grad in (("down", np.einsum("srm,srd->md", boom, d_out)), ("up", np.einsum("src,srm->cm", cat, d_pre))):
                    name = self._mlp(part, kind)
                    grads[name] = grads.get(name, 0) + grad
                d_cat = d_pre @ up.T
                d_value = d_value + d_cat[..., :d]
                back.append(d_cat[..., d:])
            d_fh_h, d_fh_t = back
        if cfg.share_feature_networks:
            grads["feature_projection"] = np.einsum("srf,srd->fd", feat, d_fh_h + d_fh_t)
        else:
            grads["head_feature_projection"] = np.einsum("srf,srd->fd", feat, d_fh_h)
            grads["tail_feature_projection"] = np.einsum("srf,srd->fd", feat, d_fh_t)
        one_net = cfg.share_feature_networks or cfg.entity_feature_size == 0
        keep.update(d_value=d_value, grads=grads, d_tails=d_tails, reg_loss=reg_loss,
                    d_feature_hidden=d_fh_h + d_fh_t if one_net else d_fh_h)
        self.last = keep
        # update (:692-704)
        self.step += 1
        alpha = adam_step_size(self.step, lr, cfg.adam_beta_m, cfg.adam_beta_v, dt)
        for name, grad in grads.items():
            mod = dt(_f32(cfg.learning_rate_modifiers.get(name, 1.0)))
            adam_update(
                self.variables[name],
                self.variables[name + "/adam_m"],
                self.variables[name + "/adam_v"],
                grad,
                alpha * mod,
                cfg,
            )
        adam_v = sqrt_v * sqrt_v
        mod = dt(_f32(cfg.learning_rate_modifiers.get("entity_embedding", 1.0)))
        adam_update(value, adam_m, adam_v, d_value, alpha * mod, cfg)
        new_rows = np.concatenate([value, adam_m, np.sqrt(adam_v), feat], axis=-1)
        for s in range(n):
            # `remote` names the padding row 0 once per padded slot.  The reference scatters all slots
            # (setEntityData, :412-417), which leaves open whose update of row 0 lasts; the slots agree
            # unless dropout gives each its own mask.  Here the first slot's update is kept.
            _, first = np.unique(remote[s], return_index=True)
            self.entity_data[s, remote[s][first]] = new_rows[s][first]
        return losses

    def train_step_loop(self, lr: float, batch: Dict[str, np.ndarray]) -> np.ndarray:
        """Mean loss per shard over the steps of one program run (:709-741).

        ``batch`` arrays carry axes ``[n_shard, n_step, ...]``.
        """
        n_step = batch["remote"].shape[1]
        total = np.zeros(self.cfg.n_shard, self.entity_data.dtype)
        for i in range(n_step):
            total += self.train_step(
                lr, *(batch[k][:, i] for k in ("remote", "a2a", "head", "relation", "tail"))
            )
        return total / self.dtype(n_step)

    # -- inference ---------------------------------------------------------

    def hidden_all(self, part: str) -> np.ndarray:
        d = self.cfg.embedding_size
        w = self.variables[self._projection(part)]
        value, fh = self.entity_data[..., :d], self.entity_data[..., 3 * d :] @ w
        if self.cfg.feature_mlp_size > 0:
            pre = np.concatenate([value, fh], axis=-1) @ self.variables[self._mlp(part, "up")]
            fh = np.maximum(pre, 0) @ self.variables[self._mlp(part, "down")]
        return value + fh

    def predict(self, shard_idx_relation: np.ndarray, shard_to_count: np.ndarray, n_best: int):
        """Brute-force ranking of every real entity for (head shard, head index, relation)
        queries; ties broken by ascending (shard, index).

        Scores follow src/poplar_kge.cpp:812-855; the reference leaves the tie
        order undefined, so the id rule is this project's own.
        Returns (shard_idx [q, n_best, 2] uint32, score [q, n_best]).
        """
        cfg = self.cfg
        q = np.asarray(shard_idx_relation).astype(np.int64)
        hid_h = self.hidden_all("head")
        hid_t = self.hidden_all("tail").reshape(-1, cfg.embedding_size)
        pred = predict_tail(cfg, hid_h[q[:, 0], q[:, 1]], self._relation_rows()[q[:, 2]])
        scores, _ = score(cfg, pred, hid_t)
        valid = np.zeros((cfg.n_shard, cfg.n_entity), bool)
        for s, count in enumerate(shard_to_count):
            valid[s, 1 : 1 + int(count)] = True
        scores = np.where(valid.reshape(1, -1), scores, -np.inf)
        order = np.argsort(-scores, axis=1, kind="stable")[:, :n_best]
        best = np.take_along_axis(scores, order, axis=1)
        shard_idx = np.stack(np.divmod(order, cfg.n_entity), axis=-1).astype(np.uint32)
        return shard_idx, best
