"""ctypes bindings and host sequencing for the CPU oracle (``soklyn_oracle.c``).

TEST INFRASTRUCTURE, NOT PRODUCT. Only the tests, the smoke check and the CPU
baseline leg of the benchmark may import this module; nothing in
``soklyn_b200`` does.

``OracleBlock`` / ``OracleFFN`` restate, on numpy f32 arrays, what the
reference's host code does around its kernels:

* ``src/io/device/ffn_device.rs:12-139``   forward of one block (GEMM, norm, act+dropout)
* ``src/io/device/ffn_device.rs:141-231``  output-layer error (zero dNorm, softmax, delta)
* ``src/io/device/ffn_device.rs:234-358``  weight gradient + optimiser step
* ``src/io/device/ffn_device.rs:360-439``  hidden-layer error then its weight step
* ``src/ffn.rs:40-57,113-166``             layer order of forward and backward
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass, field

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "liboracle.so")
_lib = None

# ordinals: src/util/function.rs:33-39,65-72,104-116,153-164; LossFunc is `as u32`.
ACT = {"identity": 0, "sigmoid": 1, "relu": 2, "leaky_relu": 3, "tanh": 4, "softmax": 5, "silu": 6, "mish": 7}
NORM = {"disabled": 0, "rms": 1, "layer": 2, "batch": 3}
LOSS = {"mse": 0, "ce": 1, "bce": 2}
REGU = {"none": 0, "l1": 1, "l2": 2}


class OkOptim(C.Structure):
    _fields_ = [("kind", C.c_uint32), ("beta1", C.c_float), ("beta2", C.c_float),
                ("epsilon", C.c_float), ("nesterov", C.c_uint32)]


def sgd(v_coeff: float = 0.0, nesterov: bool = False) -> OkOptim:
    return OkOptim(0, v_coeff, 0.0, 0.0, int(nesterov))


def adam(m_coeff: float = 0.9, v_coeff: float = 0.999, epsilon: float = 1e-8) -> OkOptim:
    return OkOptim(1, m_coeff, v_coeff, epsilon, 0)


def build(force: bool = False) -> str:
    """Compile the C restatement with gcc (OpenMP) into oracle/_build/."""
    src = os.path.join(_HERE, "soklyn_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        os.makedirs(os.path.dirname(_LIB_PATH), exist_ok=True)
        subprocess.check_call(["gcc", "-O3", "-march=x86-64-v3", "-fopenmp", "-shared", "-fPIC",
                               "-o", _LIB_PATH, src, "-lm"])
    return _LIB_PATH


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.ok_scramble_seed.restype = C.c_uint32
        _lib.ok_scramble_seed.argtypes = [C.c_uint32, C.c_uint32]
        _lib.ok_rand.restype = C.c_float
        _lib.ok_rand.argtypes = [C.c_uint32] * 3
        _lib.ok_activation.restype = C.c_float
        _lib.ok_activation.argtypes = [C.c_uint32, C.c_float, C.c_float]
        _lib.ok_activation_derivative.restype = C.c_float
        _lib.ok_activation_derivative.argtypes = [C.c_uint32] + [C.c_float] * 4
    return _lib


def _p(a):
    if a is None:
        return None
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(C.c_void_p)


def _u(v):
    return C.c_uint32(int(v))


def _f(v):
    return C.c_float(float(v))


def scramble_seed(step: int, layer_id: int) -> int:
    return int(lib().ok_scramble_seed(step & 0xFFFFFFFF, layer_id & 0xFFFFFFFF))


@dataclass
class TrainContext:
    """src/util/context.rs:40-46 (one block) / :57-74 (per-layer lists)."""
    optimiser: OkOptim
    norm_optimiser: OkOptim
    batch_size: int
    learn_rate: float
    grad_clamp: float = float(np.finfo(np.float32).max)


class OracleBlock:
    """One DenseBlock in f32 (tensor list: src/mlp.rs:268-288, :232-241, :401-411)."""

    def __init__(self, w: np.ndarray, max_batch: int, *, norm="disabled", act="identity", leaky=0.0,
                 regu="none", regu_coeff=0.0, mask_coeff=0.0, tensor_id=0, b=None):
        k, n = w.shape
        self.K, self.N, self.max_batch = k, n, max_batch
        z = lambda *s: np.zeros(s, np.float32)
        self.w = np.ascontiguousarray(w, np.float32).copy()
        self.b = z(n) if b is None else np.ascontiguousarray(b, np.float32).copy()
        self.dv_w, self.dm_w, self.dv_b, self.dm_b = z(k, n), z(k, n), z(n), z(n)
        self.norm_w, self.norm_b = np.ones(n, np.float32), z(n)
        self.dv_nw, self.dm_nw, self.dv_nb, self.dm_nb = z(n), z(n), z(n), z(n)
        self.out, self.predrop, self.preact = z(max_batch, n), z(max_batch, n), z(max_batch, n)
        self.centered, self.prenorm = z(max_batch, n), z(max_batch, n)
        self.rstd = z(max(max_batch, n))
        self.grad, self.d_prenorm = z(max_batch, n), z(max_batch, n)
        self.d_norm_w, self.d_norm_b = z(max_batch, n), z(max_batch, n)
        self.mask = np.ones((max_batch, n), np.float32)
        self.norm, self.act, self.leaky = NORM[norm], ACT[act], float(leaky)
        self.regu, self.regu_coeff = REGU[regu], float(regu_coeff)
        self.mask_coeff, self.tensor_id = float(mask_coeff), int(tensor_id)
        self.threads = 256

    # -- src/io/device/ffn_device.rs:12-139 -------------------------------------------
    def forward(self, x: np.ndarray, batch: int, use_dropout: bool, step: int,
                row_offset: int = 0) -> np.ndarray:
        L = lib()
        assert x.shape[1] == self.K and x.shape[0] >= batch and 0 < batch <= self.max_batch
        seed = scramble_seed(step, self.tensor_id)
        use_bias = self.norm != 3
        z = self.preact if self.norm == 0 else self.prenorm
        L.ok_forward_pass_0(_p(z), _p(x), _p(self.w), _p(self.b), _u(use_bias), _u(batch), _u(self.K), _u(self.N))
        if self.norm != 0:
            L.ok_forward_pass_1(_p(self.preact), _p(self.centered), _p(self.prenorm), _p(self.norm_w),
                                _p(self.norm_b), _p(self.rstd), _u(batch), _u(self.N), _u(self.norm),
                                _u(self.threads))
        L.ok_forward_pass_2(_p(self.out), _p(self.predrop), _p(self.preact), _p(self.mask), _u(batch),
                            _u(self.N), _u(self.act), _f(self.leaky), _u(use_dropout), _f(self.mask_coeff),
                            _u(seed), _u(row_offset))
        return self.out

    # -- src/io/device/ffn_device.rs:141-231 (rows = max_batch, as the reference) -------
    def compute_loss(self, target: np.ndarray, loss: str, act: str, leaky: float = 0.0, rows=None):
        L = lib()
        m = self.max_batch if rows is None else rows
        assert target.shape[0] >= m and target.shape[1] == self.N
        self.d_norm_w[:] = 0.0
        self.d_norm_b[:] = 0.0
        if ACT[act] == 5:
            L.ok_softmax(_p(self.out), _u(m), _u(self.N), _u(self.threads))
        L.ok_output_error(_p(self.out), _p(self.preact), _p(target), _p(self.norm_w), _p(self.grad),
                          _p(self.d_prenorm), _p(self.d_norm_w), _p(self.d_norm_b), _p(self.rstd),
                          _p(self.centered), _p(self.prenorm), _u(m), _u(self.N), _u(LOSS[loss]),
                          _u(self.norm), _u(ACT[act]), _f(leaky))

    # -- src/io/device/ffn_device.rs:234-358 -------------------------------------------
    def backward_output(self, x: np.ndarray, ctx: TrainContext, step: int):
        L = lib()
        assert x.shape[1] == self.K
        L.ok_backward_pass(_p(x), _p(self.w), _p(self.b), _p(self.d_prenorm), _p(self.dv_w), _p(self.dv_b),
                           _p(self.dm_w), _p(self.dm_b), _p(self.norm_w), _p(self.norm_b), _p(self.d_norm_w),
                           _p(self.d_norm_b), _p(self.dv_nw), _p(self.dv_nb), _p(self.dm_nw), _p(self.dm_nb),
                           _u(self.norm != 3), _u(self.norm), _u(ctx.batch_size), _u(self.N), _u(self.K),
                           _f(ctx.learn_rate), _f(ctx.grad_clamp), C.byref(ctx.optimiser),
                           C.byref(ctx.norm_optimiser), _u(self.regu), _f(self.regu_coeff), _u(step))

    # -- src/io/device/ffn_device.rs:360-439 -------------------------------------------
    def hidden_error(self, nxt: "OracleBlock", batch: int, m_stat=None):
        L = lib()
        assert nxt.K == self.N
        self.d_norm_w[:] = 0.0
        self.d_norm_b[:] = 0.0
        L.ok_hidden_error(_p(nxt.d_prenorm), _p(nxt.w), _p(self.norm_w), _p(self.grad), _p(self.d_prenorm),
                          _p(self.d_norm_w), _p(self.d_norm_b), _p(self.rstd), _p(self.centered),
                          _p(self.prenorm), _p(self.predrop), _p(self.preact), _p(self.mask), _u(batch),
                          _u(self.N), _u(nxt.N), _u(self.norm), _u(self.act), _f(self.leaky),
                          _u(batch if m_stat is None else m_stat))

    def backward_hidden(self, nxt: "OracleBlock", x: np.ndarray, ctx: TrainContext, step: int):
        self.hidden_error(nxt, ctx.batch_size)
        self.backward_output(x, ctx, step)

    def state(self) -> dict:
        names = ["w", "b", "dv_w", "dm_w", "dv_b", "dm_b", "norm_w", "norm_b", "dv_nw", "dm_nw", "dv_nb",
                 "dm_nb", "out", "predrop", "preact", "centered", "prenorm", "rstd", "grad", "d_prenorm",
                 "d_norm_w", "d_norm_b", "mask"]
        return {k: getattr(self, k).copy() for k in names}


class OracleFFN:
    """src/ffn.rs:10-166 — sequential stack of blocks."""

    def __init__(self, layers):
        self.layers = list(layers)

    def forward(self, x, batch, use_dropout, step, row_offset=0):
        outs, cur = [], x
        for layer in self.layers:
            cur = layer.forward(cur, batch, use_dropout, step, row_offset)
            outs.append(cur)
        return outs

    def backward(self, outputs, target, x, loss, loss_act, optimisers, norm_optimisers, batch, lr, step,
                 clamp=float(np.finfo(np.float32).max), loss_leaky=0.0):
        last = len(self.layers) - 1
        ctx = lambda i: TrainContext(optimisers[i], norm_optimisers[i], batch, lr, clamp)
        self.layers[last].compute_loss(target, loss, loss_act, loss_leaky)
        self.layers[last].backward_output(outputs[last - 1] if last > 0 else x, ctx(last), step)
        for i in range(last - 1, -1, -1):
            self.layers[i].backward_hidden(self.layers[i + 1], outputs[i - 1] if i > 0 else x, ctx(i), step)


def argmax_last(rows: np.ndarray) -> np.ndarray:
    """Row argmax where the LAST maximum wins ties (examples/mnist_train.rs:238-256,
    `max_by(partial_cmp)`)."""
    n = rows.shape[1]
    return (n - 1 - np.argmax(rows[:, ::-1], axis=1)).astype(np.int64)
