"""CPU oracle for the Pairformer triangle ops (NumPy).

TEST INFRASTRUCTURE ONLY. Nothing in the product path imports this module; it
is used by ``tests/``, by ``__graft_entry__.smoke()`` and by the CPU-baseline
legs of ``bench.py`` as the checker, never as the thing shipped or measured as
the product.

It restates, in plain NumPy, the arithmetic of the reference's XLA (jnp) path
(eightmm/FoldJAX; paths relative to its root):

* layer norm ........... src/foldjax/models/boltz2/models/primitives/_common.py:15-26
* sigmoid GLU .......... src/foldjax/models/boltz2/models/primitives/glu_backend.py:36-37
* triangle multiplication  src/foldjax/models/boltz2/models/triangle/triangle.py:78-129, 227-241
* triangle attention ... src/foldjax/models/boltz2/models/triangle/triangle_attention.py:125-162, 346-455
* pair transition ...... src/foldjax/models/boltz2/models/primitives/transition.py:99-112
* attention with pair bias  src/foldjax/models/boltz2/models/primitives/attention.py:19-140

The arithmetic itself lives in a dependency that is not vendored in the
reference: jax / jaxlib 0.10.1 (uv.lock), i.e. XLA's dot, softmax, sigmoid and
rsqrt. JAX is not installable here, so the jnp functions cannot be run.

Pinning: the reference's own tests hold complete PyTorch restatements of both
ops and assert its jnp path equals them to 2e-4 / 3e-4
(tests/models/boltz2/test_triangle_checkpoint_parity.py:155-192,
tests/models/boltz2/test_triangle_attention_checkpoint_parity.py:94-147).
``tests/golden/make_golden.py`` imports those test helpers from the reference
checkout and runs them on seeded inputs; the outputs are committed as
``tests/golden/*.npz`` and ``tests/test_oracle.py`` holds this oracle to them.
The transition is pinned the same way by the ``TorchTransition`` module of
tests/models/boltz2/test_transition_forward.py:11-33 (1e-5), the single-track attention
by ``_torch_attention_pair_bias_forward`` of
tests/models/boltz2/test_attention_checkpoint_parity.py:109-148 (2e-4).

Two precisions are offered by every function:

``dtype="float64"`` (or "float32")
    every step in that precision, no intermediate rounding: the "truth".
``dtype="bfloat16"``
    the result the reference produces for bf16 inputs: fp32 statistics and
    accumulation, with a round-to-bf16 at every point where the jnp code holds a
    bf16 array (after each matmul, each elementwise op, the LN normalisation, the
    q scaling, the attention output).
"""

from __future__ import annotations

from typing import Mapping

import numpy as np

try:  # bf16 rounding in NumPy
    import ml_dtypes

    _BF16 = ml_dtypes.bfloat16
except Exception:  # pragma: no cover - ml_dtypes ships with the image
    _BF16 = None

Params = Mapping[str, Mapping[str, np.ndarray]]


# --------------------------------------------------------------------- helpers
def round_bf16(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even to bf16, returned as float32."""
    x = np.asarray(x, dtype=np.float32)
    if _BF16 is not None:
        return x.astype(_BF16).astype(np.float32)
    u = x.view(np.uint32)
    rounded = ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
    return rounded.view(np.float32)


class _Prec:
    """Working precision plus the rounding applied where the reference holds the trunk dtype."""

    def __init__(self, dtype: str):
        if dtype not in ("float64", "float32", "bfloat16"):
            raise ValueError(f"unsupported oracle dtype: {dtype!r}")
        self.name = dtype
        self.work = np.float64 if dtype == "float64" else np.float32
        self.bf16 = dtype == "bfloat16"

    def r(self, x: np.ndarray) -> np.ndarray:
        return round_bf16(x) if self.bf16 else np.asarray(x, dtype=self.work)

    def arr(self, x) -> np.ndarray:
        return self.r(np.asarray(x, dtype=np.float32 if self.bf16 else self.work))


def _sigmoid(x: np.ndarray) -> np.ndarray:
    """Overflow-free logistic: 1 / (1 + exp(-x)) for x >= 0 and exp(x) / (1 + exp(x)) below."""
    e = np.exp(-np.abs(x))
    return np.where(x >= 0, 1.0 / (1.0 + e), e / (1.0 + e)).astype(x.dtype, copy=False)


def layer_norm(x: np.ndarray, scale: np.ndarray, bias: np.ndarray, eps: float, dtype: str = "float64") -> np.ndarray:
    """_common.py:15-26: fp32 statistics, biased variance, the normalised value
    cast to the input dtype BEFORE the affine step, which runs in that dtype."""
    pr = _Prec(dtype)
    xf = pr.arr(x)
    mean = xf.mean(axis=-1, keepdims=True, dtype=pr.work)
    var = np.square(xf - mean).mean(axis=-1, keepdims=True, dtype=pr.work)
    normed = pr.r((xf - mean) / np.sqrt(var + pr.work(eps)))
    return pr.r(pr.r(normed * pr.arr(scale)) + pr.arr(bias))


def _linear(x: np.ndarray, kernel: np.ndarray, pr: _Prec) -> np.ndarray:
    """x @ kernel with the kernel in [in, out] layout; fp32 accumulate, output in the trunk dtype."""
    return pr.r(np.matmul(x, pr.arr(kernel)))


# ------------------------------------------------------- triangle multiplication
def triangle_multiplication(
    params: Params,
    x: np.ndarray,
    mask: np.ndarray | None,
    direction: str,
    eps: float = 1e-5,
    dtype: str = "float64",
) -> np.ndarray:
    """triangle.py:78-129 (XLA path, contraction_precision="float32").

    x [B,N,N,C], mask [B,N,N] -> update [B,N,N,C] (the caller adds the residual).
    """
    if direction not in ("outgoing", "incoming"):
        raise ValueError(f"Unsupported triangle multiplication direction: {direction!r}")
    pr = _Prec(dtype)
    xn = layer_norm(x, params["norm_in"]["scale"], params["norm_in"]["bias"], eps, dtype)  # :78
    x_in = xn
    if mask is None:
        mask = np.ones(xn.shape[:-1], dtype=pr.work)
    m = pr.arr(mask)
    gate = pr.r(_sigmoid(_linear(xn, params["g_in"]["kernel"], pr)))  # glu_backend.py:36-37
    projected = pr.r(gate * _linear(xn, params["p_in"]["kernel"], pr))
    projected = pr.r(projected * m[..., None])  # :90
    a, b = np.split(projected.astype(pr.work), 2, axis=-1)  # :96-102, a = first half
    # channel-major batched matmuls (BLAS) instead of a generic einsum; same sums
    at = np.ascontiguousarray(np.transpose(a, (0, 3, 1, 2)))  # [b, d, row, col]
    bt = np.ascontiguousarray(np.transpose(b, (0, 3, 1, 2)))
    if direction == "outgoing":
        out = np.matmul(at, np.swapaxes(bt, -1, -2))  # "bikd,bjkd->bijd"  :231
    else:
        out = np.matmul(np.swapaxes(at, -1, -2), bt)  # "bkid,bkjd->bijd"  :239
    out = pr.r(np.transpose(out, (0, 2, 3, 1)))  # :124
    out = layer_norm(out, params["norm_out"]["scale"], params["norm_out"]["bias"], eps, dtype)  # :126
    out = _linear(out, params["p_out"]["kernel"], pr)  # :127
    g = pr.r(_sigmoid(_linear(x_in, params["g_out"]["kernel"], pr)))  # :128
    return pr.r(out * g)  # :129


def triangle_contraction(a: np.ndarray, b: np.ndarray, direction: str) -> np.ndarray:
    """triangle.py:227-241 on [N,N,C] operands, float64."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    if direction == "outgoing":
        return np.einsum("ikd,jkd->ijd", a, b, optimize=True)
    return np.einsum("kid,kjd->ijd", a, b, optimize=True)


# ------------------------------------------------------------ triangle attention
def attention_core(
    q: np.ndarray,
    k: np.ndarray,
    v: np.ndarray,
    tri_bias: np.ndarray,
    mask_bias: np.ndarray,
    dtype: str = "float64",
    row_chunk: int = 16,
    threads: int | None = None,
) -> np.ndarray:
    """triangle_attention.py:428-455.

    q,k,v [B,I,H,J,D] (q pre-scaled); tri_bias [B,1,H,J,J]; mask_bias [B,I,1,1,J]
    additive (0 / -inf constant). scores = (q k^T + mask_bias) + tri_bias in the
    working precision, softmax, P v, cast to the trunk dtype. Rows are chunked
    only to bound memory; rows are independent so the result is unchanged.
    """
    pr = _Prec(dtype)
    work = pr.work
    q = np.asarray(q, dtype=work)
    k = np.asarray(k, dtype=work)
    v = np.asarray(v, dtype=work)
    tb = np.asarray(tri_bias, dtype=work)
    mb = np.asarray(mask_bias, dtype=work)
    out = np.empty_like(q)
    n_i = q.shape[1]

    def rows(s: int) -> None:
        e = min(n_i, s + row_chunk)
        scores = np.matmul(q[:, s:e], np.swapaxes(k[:, s:e], -1, -2))
        scores = scores + mb[:, s:e] + tb  # that order: :453
        scores = scores - scores.max(axis=-1, keepdims=True)
        p = np.exp(scores)
        p /= p.sum(axis=-1, keepdims=True)
        out[:, s:e] = np.matmul(p, v[:, s:e])

    starts = range(0, n_i, row_chunk)
    if threads and threads > 1 and len(starts) > 1:  # rows are independent; NumPy releases the GIL in these ops
        from concurrent.futures import ThreadPoolExecutor

        with ThreadPoolExecutor(max_workers=threads) as pool:
            list(pool.map(rows, starts))
    else:
        for s in starts:
            rows(s)
    return pr.r(out)


def triangle_attention(
    params: Params,
    x: np.ndarray,
    mask: np.ndarray | None = None,
    starting: bool = True,
    inf: float = 1e9,
    eps: float = 1e-5,
    dtype: str = "float64",
    return_parts: bool = False,
    threads: int | None = None,
):
    """triangle_attention.py:79-162 and 346-425 (XLA path).

    x [B,N,N,C], mask [B,N,N] -> update [B,N,N,C]. Heads come from the bias
    projection's width, head dim from linear_g's.
    """
    pr = _Prec(dtype)
    work = pr.work
    xx = pr.arr(x)
    if mask is None:
        mask = np.ones(xx.shape[:-1], dtype=work)
    m = np.asarray(mask, dtype=work)
    if not starting:  # :128-130
        xx = np.swapaxes(xx, -2, -3)
        m = np.swapaxes(m, -1, -2)
    xn = layer_norm(xx, params["layer_norm"]["scale"], params["layer_norm"]["bias"], eps, dtype)  # :132
    # :138-142 - built in fp32 so the constant stays finite
    mask_bias = (np.float32(inf) * (m.astype(np.float32) - np.float32(1.0)))[:, :, None, None, :]
    tri_bias = _linear(xn, params["linear"]["kernel"], pr)  # [B,J,K,H]  :144
    heads = tri_bias.shape[-1]
    tri_bias = np.transpose(tri_bias, (0, 3, 1, 2))[:, None]  # [B,1,H,J,K]  :145-146

    mha = params["mha"]
    qg = _linear(xn, np.concatenate((mha["linear_q"]["kernel"], mha["linear_g"]["kernel"]), axis=-1), pr)  # :360
    q, gate = np.split(qg, 2, axis=-1)
    kv = _linear(xn, np.concatenate((mha["linear_k"]["kernel"], mha["linear_v"]["kernel"]), axis=-1), pr)  # :368
    k, v = np.split(kv, 2, axis=-1)
    c_hidden = np.asarray(mha["linear_g"]["kernel"]).shape[-1] // heads

    def heads_first(t):  # [B,I,J,H*D] -> [B,I,H,J,D]   :377-382
        t = t.reshape(t.shape[:-1] + (heads, c_hidden))
        return np.swapaxes(t, -2, -3)

    q, k, v = heads_first(q), heads_first(k), heads_first(v)
    q_scale = pr.r(np.sqrt(np.asarray(c_hidden, dtype=work)))  # sqrt evaluated in the trunk dtype  :399
    q = pr.r(q / q_scale)  # :400
    o = attention_core(q, k, v, tri_bias, mask_bias, dtype, threads=threads)  # :414
    o = np.swapaxes(o, -2, -3)  # [B,I,J,H,D]
    g = pr.r(_sigmoid(gate)).reshape(gate.shape[:-1] + (heads, c_hidden))  # :421-422
    o = pr.r(o * g)
    o = o.reshape(o.shape[:-2] + (heads * c_hidden,))
    out = _linear(o, mha["linear_o"]["kernel"], pr)  # :425
    if not starting:  # :160-161
        out = np.swapaxes(out, -2, -3)
    if return_parts:
        return out, {"q": q, "k": k, "v": v, "tri_bias": tri_bias, "mask_bias": mask_bias, "gate": g}
    return out


# ---------------------------------------------- sampled elements of large cases
def triangle_multiplication_sampled(
    params: Params,
    xi: np.ndarray,
    mi: np.ndarray | None,
    xj: np.ndarray,
    mj: np.ndarray | None,
    xij: np.ndarray,
    eps: float = 1e-5,
    dtype: str = "float64",
) -> np.ndarray:
    """Elements ``update[i_r, j_s, :]`` of triangle_multiplication (triangle.py:78-129)
    for sampled rows i_r and columns j_s, without forming the whole tensor.

    ``out[i, j] = sum_k a[i, k] * b[j, k]`` (outgoing) needs only rows i and j of the
    input; the incoming direction is the same sum over the transposed input. So the
    caller passes, in the frame where k runs along axis 1,

        xi [R, N, C], mi [R, N]   x[i_r, :] and its mask row  (incoming: x[:, i_r], mask[:, i_r])
        xj [S, N, C], mj [S, N]   x[j_s, :]                   (incoming: x[:, j_s], mask[:, j_s])
        xij [R, S, C]             x[i_r, j_s], the pair the output gate is computed from

    and gets ``[R, S, C]``. Same rounding points as the full restatement."""
    pr = _Prec(dtype)

    def project(x, m):
        xn = layer_norm(x, params["norm_in"]["scale"], params["norm_in"]["bias"], eps, dtype)
        gate = pr.r(_sigmoid(_linear(xn, params["g_in"]["kernel"], pr)))
        proj = pr.r(gate * _linear(xn, params["p_in"]["kernel"], pr))
        if m is not None:
            proj = pr.r(proj * pr.arr(m)[..., None])
        return proj.astype(pr.work)

    c = np.asarray(params["p_out"]["kernel"]).shape[0]
    a = project(xi, mi)[..., :c]  # a = first half of the projection  :102
    b = project(xj, mj)[..., c:]
    out = pr.r(np.einsum("rkd,skd->rsd", a, b, optimize=True))  # :231 / :239, :124
    out = layer_norm(out, params["norm_out"]["scale"], params["norm_out"]["bias"], eps, dtype)
    out = _linear(out, params["p_out"]["kernel"], pr)
    x_in = layer_norm(xij, params["norm_in"]["scale"], params["norm_in"]["bias"], eps, dtype)
    g = pr.r(_sigmoid(_linear(x_in, params["g_out"]["kernel"], pr)))
    return pr.r(out * g)


def triangle_attention_sampled(
    params: Params,
    xi: np.ndarray,
    mi: np.ndarray | None,
    xj: np.ndarray,
    cols: np.ndarray,
    inf: float = 1e9,
    eps: float = 1e-5,
    dtype: str = "float64",
) -> np.ndarray:
    """Elements ``update[i_r, j_s, :]`` of the starting-node triangle attention
    (triangle_attention.py:79-162, 346-455) for sampled rows i_r and queries j_s.

    Row i attends over the keys of its own row with the bias ``LN(x)[j, k] @ W``, so the
    sampled elements need only rows i_r and j_s of the input:

        xi [R, N, C], mi [R, N]   x[i_r, :] and mask[i_r, :]   (ending node: x[:, i_r], mask[:, i_r])
        xj [S, N, C]              x[j_s, :]                    (ending node: x[:, j_s])
        cols [S]                  the indices j_s (the queries inside row i)

    Returns ``[R, S, C]``."""
    pr = _Prec(dtype)
    work = pr.work
    cols = np.asarray(cols)
    xn_i = layer_norm(pr.arr(xi), params["layer_norm"]["scale"], params["layer_norm"]["bias"], eps, dtype)
    xn_j = layer_norm(pr.arr(xj), params["layer_norm"]["scale"], params["layer_norm"]["bias"], eps, dtype)
    n = xn_i.shape[1]
    m = np.ones(xn_i.shape[:2], dtype=np.float32) if mi is None else np.asarray(mi, dtype=np.float32)
    mask_bias = (np.float32(inf) * (m - np.float32(1.0))).astype(work)  # [R, K]
    tri_bias = np.transpose(_linear(xn_j, params["linear"]["kernel"], pr), (2, 0, 1))  # [H, S, K]
    heads = tri_bias.shape[0]
    mha = params["mha"]
    c_hidden = np.asarray(mha["linear_g"]["kernel"]).shape[-1] // heads
    xq = xn_i[:, cols]  # [R, S, C]: the sampled queries of every sampled row
    qg = _linear(xq, np.concatenate((mha["linear_q"]["kernel"], mha["linear_g"]["kernel"]), axis=-1), pr)
    q, gate = np.split(qg, 2, axis=-1)
    kv = _linear(xn_i, np.concatenate((mha["linear_k"]["kernel"], mha["linear_v"]["kernel"]), axis=-1), pr)
    k, v = np.split(kv, 2, axis=-1)
    split = lambda t: np.swapaxes(t.reshape(t.shape[:-1] + (heads, c_hidden)), -2, -3)  # [R, H, *, D]
    q, k, v = split(q), split(k), split(v)
    q_scale = pr.r(np.sqrt(np.asarray(c_hidden, dtype=work)))
    q = pr.r(q / q_scale).astype(work)
    scores = np.matmul(q, np.swapaxes(k.astype(work), -1, -2))  # [R, H, S, K]
    scores = scores + mask_bias[:, None, None, :] + tri_bias[None].astype(work)
    scores = scores - scores.max(axis=-1, keepdims=True)
    p = np.exp(scores)
    p /= p.sum(axis=-1, keepdims=True)
    o = pr.r(np.matmul(p, v.astype(work)))  # [R, H, S, D]
    o = np.swapaxes(o, -2, -3)  # [R, S, H, D]
    g = pr.r(_sigmoid(gate)).reshape(gate.shape[:-1] + (heads, c_hidden))
    o = pr.r(o * g).reshape(o.shape[:-2] + (heads * c_hidden,))
    assert o.shape[1] == len(cols) and n == xn_j.shape[1]
    return _linear(o, mha["linear_o"]["kernel"], pr)


# ------------------------------------------------------------- pair transition
def transition(params: Params, x: np.ndarray, eps: float = 1e-5, dtype: str = "float64") -> np.ndarray:
    """transition.py:99-112 (the unchunked XLA branch): LN, one matmul against
    concat(fc1, fc2), silu(first half) * second half, matmul against fc3.
    x [..., C] -> update [..., C] (the caller adds the residual,
    pairformer.py:152-160). In bf16 the matmul outputs, the sigmoid and both
    products are each rounded to the trunk dtype."""
    pr = _Prec(dtype)
    xn = layer_norm(x, params["norm"]["scale"], params["norm"]["bias"], eps, dtype)  # :99
    a = _linear(xn, params["fc1"]["kernel"], pr)  # :108-109
    b = _linear(xn, params["fc2"]["kernel"], pr)
    silu = pr.r(a * pr.r(_sigmoid(a)))  # jax.nn.silu = x * sigmoid(x)  :110
    hidden = pr.r(silu * b)
    return _linear(hidden, params["fc3"]["kernel"], pr)  # :111


def random_transition_params(rng: np.random.Generator, c_z: int = 128, expansion: int = 4, std: float = 0.02,
                             ln_noise: float = 0.0) -> dict:
    def w(*shape):
        return (rng.standard_normal(shape) * std).astype(np.float32)

    hidden = expansion * c_z
    return {
        "norm": {
            "scale": (1.0 + ln_noise * rng.standard_normal(c_z)).astype(np.float32),
            "bias": (ln_noise * rng.standard_normal(c_z)).astype(np.float32),
        },
        "fc1": {"kernel": w(c_z, hidden)},
        "fc2": {"kernel": w(c_z, hidden)},
        "fc3": {"kernel": w(hidden, c_z)},
    }


# ------------------------------------------------ single attention with pair bias
def attention_pair_bias(params: Params, s: np.ndarray, z: np.ndarray, mask: np.ndarray, k_in: np.ndarray | None = None,
                        inf: float = 1e6, eps: float = 1e-5, dtype: str = "float64") -> np.ndarray:
    """attention.py:19-140 (XLA path), as the Pairformer block calls it
    (trunk_blocks/pairformer.py:188-203): s [B,N,c_s] (already layer-normed by the
    caller) and z [B,N,N,c_z] arrive in float32 whatever the trunk dtype, so there is
    no bf16 mode: ``dtype`` is "float64" or "float32". mask [B,N] -> [B,N,c_s]."""
    if dtype not in ("float64", "float32"):
        raise ValueError("the single-track attention runs in float32 in the reference; use float64 or float32")
    work = np.float64 if dtype == "float64" else np.float32
    f = lambda name, leaf="kernel": np.asarray(params[name][leaf], dtype=work)
    s = np.asarray(s, dtype=work)
    k_in = s if k_in is None else np.asarray(k_in, dtype=work)
    batch, n, c_s = s.shape
    heads = f("proj_z").shape[-1]
    hd = c_s // heads
    q = (s @ f("proj_q") + f("proj_q", "bias")).reshape(batch, n, heads, hd)  # :46-52
    g = _sigmoid(s @ f("proj_g"))  # :53
    k = (k_in @ f("proj_k")).reshape(batch, -1, heads, hd)  # :54-62
    v = (k_in @ f("proj_v")).reshape(batch, -1, heads, hd)
    zf = np.asarray(z, dtype=work)
    mean = zf.mean(-1, keepdims=True)
    var = np.square(zf - mean).mean(-1, keepdims=True)
    zn = (zf - mean) / np.sqrt(var + work(eps)) * f("proj_z_norm", "scale") + f("proj_z_norm", "bias")  # :64-69
    bias = np.transpose(zn @ f("proj_z"), (0, 3, 1, 2))  # [B,H,N,N]  :70-71
    mask_bias = (1.0 - np.asarray(mask, dtype=work))[:, None, None, :] * work(-inf)  # :92
    attn = np.einsum("bihd,bjhd->bhij", q, k) / np.sqrt(work(hd)) + bias + mask_bias  # :134-136
    attn = attn - attn.max(-1, keepdims=True)
    attn = np.exp(attn)
    attn = attn / attn.sum(-1, keepdims=True)
    out = np.einsum("bhij,bjhd->bihd", attn, v).reshape(batch, n, c_s)
    return (g * out) @ f("proj_o")  # :116-117


def random_attention_pair_bias_params(rng: np.random.Generator, c_s: int = 384, c_z: int = 128, heads: int = 16,
                                      std: float = 0.02, ln_noise: float = 0.0) -> dict:
    def w(*shape):
        return (rng.standard_normal(shape) * std).astype(np.float32)

    return {
        "proj_q": {"kernel": w(c_s, c_s), "bias": w(c_s)},
        "proj_k": {"kernel": w(c_s, c_s)},
        "proj_v": {"kernel": w(c_s, c_s)},
        "proj_g": {"kernel": w(c_s, c_s)},
        "proj_z_norm": {"scale": (1.0 + ln_noise * rng.standard_normal(c_z)).astype(np.float32),
                        "bias": (ln_noise * rng.standard_normal(c_z)).astype(np.float32)},
        "proj_z": {"kernel": w(c_z, heads)},
        "proj_o": {"kernel": w(c_s, c_s)},
    }


# ------------------------------------------------------------- one Pairformer block
def pairformer_layer(params: Params, s: np.ndarray | None, z: np.ndarray, mask: np.ndarray | None,
                     pair_mask: np.ndarray | None, eps: float = 1e-5, dtype: str = "float64", *,
                     pair_gate: bool = False, mask_transition: bool = False, attention_first: bool = False):
    """pairformer_layer_forward, trunk_blocks/pairformer.py:126-206: the four triangle updates
    and the pair transition on z (trunk dtype, residual sums rounded to it), then the single
    track in float32 (float64 here when ``dtype`` is "float64"): s += attention_pair_bias(LN(s),
    z) ; s += transition_s(s). s = None runs the pair track only. Returns (s, z).

    Block variants of the other model families, on the same op arithmetic:
    ``pair_gate`` - Protenix's block (protenix/models/trunk_blocks/pairformer.py:71-180): z is
    multiplied by (pair_mask != 0) first and after every update, s by the token gate (the
    diagonal of the pair mask unless ``mask`` is given) first and after both of its updates;
    ``mask_transition`` - OpenFold3's pair block (openfold3/models/pair_block.py:174-183): the
    pair transition's update is multiplied by the pair mask;
    ``attention_first`` - its ``tri_mul_first=False`` order (pair_block.py:151-171)."""
    pr = _Prec(dtype)
    z = pr.arr(z)
    gate_z = None
    if pair_gate and pair_mask is not None:
        gate_z = (np.asarray(pair_mask) != 0).astype(z.dtype)[..., None]
        z = z * gate_z
        if mask is None:
            mask = np.diagonal(np.asarray(pair_mask) != 0, axis1=-2, axis2=-1).astype(np.float32)

    def gated(v):
        return v if gate_z is None else v * gate_z

    mults = (lambda v: triangle_multiplication(params["tri_mul_out"], v, pair_mask, "outgoing", eps, dtype),
             lambda v: triangle_multiplication(params["tri_mul_in"], v, pair_mask, "incoming", eps, dtype))
    atts = (lambda v: triangle_attention(params["tri_att_start"], v, pair_mask, True, eps=eps, dtype=dtype),
            lambda v: triangle_attention(params["tri_att_end"], v, pair_mask, False, eps=eps, dtype=dtype))
    for update in (atts + mults if attention_first else mults + atts):
        z = gated(pr.r(z + update(z)))
    upd = transition(params["transition_z"], z, eps, dtype)
    if mask_transition and pair_mask is not None:
        upd = pr.r(upd * pr.r(np.asarray(pair_mask, dtype=upd.dtype))[..., None])
    z = gated(pr.r(z + upd))
    if s is None:
        return None, z
    wide = "float64" if dtype == "float64" else "float32"
    work = np.float64 if wide == "float64" else np.float32
    s = np.asarray(s, dtype=work)
    if mask is None:
        mask = np.ones(s.shape[:2], dtype=work)
    gate_s = (np.asarray(mask) != 0).astype(work)[..., None] if gate_z is not None else None
    if gate_s is not None:
        s = s * gate_s
    s_normed = layer_norm(s, params["pre_norm_s"]["scale"], params["pre_norm_s"]["bias"], eps, wide)
    s = s + attention_pair_bias(params["attention"], s_normed, z, mask, k_in=s_normed, eps=eps, dtype=wide)
    if gate_s is not None:
        s = s * gate_s
    s = s + transition(params["transition_s"], s, eps, wide)
    if gate_s is not None:
        s = s * gate_s
    return s, z


def random_pairformer_params(rng: np.random.Generator, c_s: int = 384, heads_s: int = 16, std: float = 0.02,
                             ln_noise: float = 0.0) -> dict:
    ln = lambda c: {"scale": (1.0 + ln_noise * rng.standard_normal(c)).astype(np.float32),
                    "bias": (ln_noise * rng.standard_normal(c)).astype(np.float32)}
    w = lambda *shape: (rng.standard_normal(shape) * std).astype(np.float32)
    return {
        "tri_mul_out": random_trimul_params(rng, std=std, ln_noise=ln_noise),
        "tri_mul_in": random_trimul_params(rng, std=std, ln_noise=ln_noise),
        "tri_att_start": random_triatt_params(rng, std=std, ln_noise=ln_noise),
        "tri_att_end": random_triatt_params(rng, std=std, ln_noise=ln_noise),
        "transition_z": random_transition_params(rng, std=std, ln_noise=ln_noise),
        "pre_norm_s": ln(c_s),
        "attention": random_attention_pair_bias_params(rng, c_s=c_s, heads=heads_s, std=std, ln_noise=ln_noise),
        "transition_s": {"norm": ln(c_s), "fc1": {"kernel": w(c_s, 4 * c_s)}, "fc2": {"kernel": w(c_s, 4 * c_s)},
                         "fc3": {"kernel": w(4 * c_s, c_s)}},
    }


# ------------------------------------------------------------ synthetic inputs
def random_trimul_params(rng: np.random.Generator, c_z: int = 128, c_hidden: int = 128, std: float = 0.02,
                         ln_noise: float = 0.0) -> dict:
    """Weights as the benchmark configs describe them: N(0, std^2) linear kernels
    in [in, out] layout, layer-norm scale 1 / bias 0 (optionally perturbed so
    that tests exercise the affine step)."""

    def w(*shape):
        return (rng.standard_normal(shape) * std).astype(np.float32)

    def ln(c):
        return {
            "scale": (1.0 + ln_noise * rng.standard_normal(c)).astype(np.float32),
            "bias": (ln_noise * rng.standard_normal(c)).astype(np.float32),
        }

    return {
        "norm_in": ln(c_z),
        "p_in": {"kernel": w(c_z, 2 * c_hidden)},
        "g_in": {"kernel": w(c_z, 2 * c_hidden)},
        "norm_out": ln(c_hidden),
        "p_out": {"kernel": w(c_hidden, c_z)},
        "g_out": {"kernel": w(c_z, c_z)},
    }


def random_triatt_params(rng: np.random.Generator, c_z: int = 128, heads: int = 4, c_hidden: int = 32,
                         std: float = 0.02, ln_noise: float = 0.0) -> dict:
    def w(*shape):
        return (rng.standard_normal(shape) * std).astype(np.float32)

    hd = heads * c_hidden
    return {
        "layer_norm": {
            "scale": (1.0 + ln_noise * rng.standard_normal(c_z)).astype(np.float32),
            "bias": (ln_noise * rng.standard_normal(c_z)).astype(np.float32),
        },
        "linear": {"kernel": w(c_z, heads)},
        "mha": {
            "linear_q": {"kernel": w(c_z, hd)},
            "linear_k": {"kernel": w(c_z, hd)},
            "linear_v": {"kernel": w(c_z, hd)},
            "linear_g": {"kernel": w(c_z, hd)},
            "linear_o": {"kernel": w(hd, c_z)},
        },
    }


def round_params(params, dtype: str):
    """Round every leaf to the trunk dtype (what a bf16 checkpoint cast does)."""
    if dtype != "bfloat16":
        return params
    if isinstance(params, Mapping):
        return {k: round_params(v, dtype) for k, v in params.items()}
    return round_bf16(params)


def pad_mask(n: int, n_pad: int) -> np.ndarray:
    """pair mask m m^T with the last n_pad tokens dropped, shape [1, n, n]."""
    m = np.ones(n, dtype=np.float32)
    if n_pad:
        m[n - n_pad:] = 0.0
    return (m[:, None] * m[None, :])[None]


def error_vs(ref: np.ndarray, got: np.ndarray) -> dict:
    """The benchmark's error framing: max-abs and mean-abs error relative to the
    RMS of the reference output (the reference's own scripts report the same,
    tests/models/boltz2/scripts/compare_trunk_backends.py:25-40)."""
    ref = np.asarray(ref, dtype=np.float64)
    got = np.asarray(got, dtype=np.float64)
    rms = float(np.sqrt(np.mean(np.square(ref)))) or 1.0
    diff = np.abs(ref - got)
    return {"max_abs_over_rms": float(diff.max() / rms), "mean_abs_over_rms": float(diff.mean() / rms), "rms": rms}
