"""pyre_b200: host-side mirror of the reference's Qwen-Next model surface over the C ABI.

The product is the shared library ``libpyre_b200.so`` (hand-written sm_100a CUDA kernels
behind ``include/pyre_b200.h``).  This module is a thin ctypes layer whose classes carry
the names and call shapes of the reference's Rust items (``QMat::matmul``,
``Model::forward`` / ``forward_multi`` / ``spec_keep``, ``State``), so tests and
benchmarks read like the reference's own code.  There is no CPU fallback: importing works
anywhere, but creating a :class:`Ctx` without the library or without a GPU raises.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "libpyre_b200.so"

# ggml type ids (QType::from_id, src/model/gguf_q.rs:23-29 of the reference)
F32, F16, Q8_0, Q4_K, IQ2_XS, IQ3_S, BF16 = 0, 1, 8, 12, 17, 21, 30
IQ3_XXS, IQ4_NL, IQ2_S, IQ4_XS = 18, 20, 22, 23          # the further formats of mixed-type files
Q6_K, IQ2_XXS, Q2_0, IQ1_M = 14, 16, 42, 29
Q4_0, Q5_0, Q3_K, Q5_K = 2, 6, 11, 13
TYPE_NAMES = {"F32": F32, "F16": F16, "Q8_0": Q8_0, "Q4_K": Q4_K, "IQ2_XS": IQ2_XS, "IQ3_S": IQ3_S, "BF16": BF16,
              "IQ3_XXS": IQ3_XXS, "IQ4_NL": IQ4_NL, "IQ2_S": IQ2_S, "IQ4_XS": IQ4_XS,
              "Q6_K": Q6_K, "IQ2_XXS": IQ2_XXS, "Q2_0": Q2_0, "IQ1_M": IQ1_M, "Q4_0": Q4_0, "Q5_0": Q5_0, "Q3_K": Q3_K, "Q5_K": Q5_K}

PB_OK, PB_ERR_ARG, PB_ERR_CUDA, PB_ERR_OOM, PB_UNSUPPORTED, PB_ERR_DEVICE, PB_ERR_STATE = range(7)
_STATUS = {1: "PB_ERR_ARG", 2: "PB_ERR_CUDA", 3: "PB_ERR_OOM", 4: "PB_UNSUPPORTED", 5: "PB_ERR_DEVICE", 6: "PB_ERR_STATE"}

ROLES = [
    "TOKEN_EMBD", "OUTPUT", "OUT_NORM", "ATTN_NORM", "FFN_NORM",
    "ATTN_Q", "ATTN_K", "ATTN_V", "ATTN_O", "ATTN_Q_NORM", "ATTN_K_NORM",
    "LIN_QKV", "LIN_Z", "LIN_BETA", "LIN_ALPHA", "LIN_OUT", "LIN_A", "LIN_DT", "LIN_CONV", "LIN_NORM",
    "ROUTER", "EXP_GATE", "EXP_UP", "EXP_DOWN", "SH_GATE", "SH_UP", "SH_DOWN", "SH_GATE_INP",
    "HCA_NORM", "HCA_DOWN", "HCA_UP", "HCA_INJECT", "HCF_NORM", "HCF_DOWN", "HCF_UP", "HCF_INJECT",
    "OUT_HC_NORM", "OUT_HC_DOWN", "OUT_HC_UP",
    "IDX_Q", "IDX_K", "IDX_Q_NORM", "IDX_K_NORM",
    "MTP_FC_E", "MTP_FC_H", "MTP_PRE_E", "MTP_PRE_H",
    "PLE_TAB", "PLE_KEY", "PLE_VALUE", "PLE_NORM_KEY", "PLE_NORM_QUERY", "PLE_NORM_CONV", "PLE_CONV",
]
ROLE = {n: i for i, n in enumerate(ROLES)}


class PyreError(RuntimeError):
    def __init__(self, status: int, msg: str):
        super().__init__(f"{_STATUS.get(status, status)}: {msg}")
        self.status = status


class Cfg(C.Structure):
    """Cfg, src/model/qwen4exp_gguf.rs:18-26 (decode-path fields)."""
    _fields_ = [(n, C.c_int32) for n in ("n_layers", "d", "hc", "hc_lr", "n_head", "n_kv", "hd", "n_rot")] + \
               [("rope_base", C.c_float), ("eps", C.c_float)] + \
               [(n, C.c_int32) for n in ("n_exp", "top_k", "ff_exp", "ff_sh", "lin_nk", "lin_nv", "lin_dk", "lin_dv",
                                         "conv_k", "full_every", "vocab", "max_ctx", "kv_bits", "kv_recent")]


class Caps(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("multi_ok", "max_window", "max_ctx", "max_batch", "ep_world")]


class Stats(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("steps", "kernels_launched", "weight_bytes_per_step", "kv_bytes_per_step", "state_bytes_per_step", "device_ns", "exchange_ns")]


def make_cfg(**kw) -> Cfg:
    """Defaults of the benchmark model (hidden 2048, 16:2 heads of 256, 512 experts top-10, DeltaNet 16/32 x 128)."""
    c = Cfg()
    d = dict(n_layers=4, d=2048, hc=0, hc_lr=0, n_head=16, n_kv=2, hd=256, n_rot=64, rope_base=1e7, eps=1e-6,
             n_exp=512, top_k=10, ff_exp=512, ff_sh=512, lin_nk=16, lin_nv=32, lin_dk=128, lin_dv=128,
             conv_k=4, full_every=4, vocab=151936, max_ctx=4096, kv_bits=0, kv_recent=1024)
    d.update(kw)
    for k, v in d.items():
        setattr(c, k, v)
    return c


_lib = None


def lib():
    """Load libpyre_b200.so; raises if it has not been built (no fallback)."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(f"{LIB_PATH} is missing: build it with `python -m pyre_b200.build` (nvcc, sm_100a)")
        L = C.CDLL(str(LIB_PATH))
        L.pb_last_error.restype = C.c_char_p
        L.pb_last_error.argtypes = [C.c_void_p]
        _lib = L
    return _lib


def _p(a):
    if a is None:
        return None
    if isinstance(a, np.ndarray):
        return a.ctypes.data_as(C.c_void_p)
    return C.c_void_p(int(a))


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


class Ctx:
    """One GPU, one worker thread (the reference's Cube, src/model/qn_cube.rs:6237-6250)."""

    def __init__(self, device: int = 0):
        self.h = C.c_void_p()
        rc = lib().pb_ctx_create(C.c_int(device), C.byref(self.h))
        if rc:
            raise PyreError(rc, "pb_ctx_create failed (is a CUDA device visible?)")
        self.device = device

    def check(self, rc: int):
        if rc:
            raise PyreError(rc, lib().pb_last_error(self.h).decode())

    def set_stream(self, cuda_stream: int):
        """Launch on this cudaStream_t (0 = legacy default stream)."""
        self.check(lib().pb_ctx_set_stream(self.h, C.c_void_p(cuda_stream)))

    def own_stream(self):
        self.check(lib().pb_ctx_own_stream(self.h))

    def pinned_empty(self, shape, dtype=np.float32) -> np.ndarray:
        """An array in page-locked host memory (pb_host_alloc): logits read into it take one DMA instead of a staging copy and a
        host copy.  The memory is released when the array (and every view of it) is gone."""
        shape = tuple(int(x) for x in (shape if isinstance(shape, (tuple, list)) else (shape,)))
        n = int(np.prod(shape, dtype=np.int64)) * np.dtype(dtype).itemsize
        ptr = C.c_void_p()
        self.check(lib().pb_host_alloc(self.h, C.c_size_t(n), C.byref(ptr)))
        buf = (C.c_uint8 * max(n, 1)).from_address(ptr.value)
        arr = np.frombuffer(buf, dtype=np.uint8, count=n).view(dtype).reshape(shape)
        free = lib().pb_host_free
        import weakref
        weakref.finalize(buf, lambda a=ptr.value: free(None, C.c_void_p(a)))     # without the context: the array may outlive it
        return arr

    def sync(self):
        self.check(lib().pb_ctx_sync(self.h))

    def device_status(self) -> int:
        st = C.c_int()
        self.check(lib().pb_ctx_device_status(self.h, C.byref(st)))
        return st.value

    def poll(self) -> bool:
        """True while work of this context is still running on the GPU (pb_poll); raises on a reported device failure."""
        busy = C.c_int()
        self.check(lib().pb_poll(self.h, C.byref(busy)))
        return bool(busy.value)

    def stamps_enable(self, slots: int):
        self.check(lib().pb_ctx_stamps_enable(self.h, C.c_int(slots)))

    def stamps_read(self, max_slots: int = 8192):
        """(stamps [n][8] uint64 nanoseconds, kernel ids [n]) of the launches traced so far."""
        st = np.zeros((max_slots, 8), dtype=np.uint64)
        ids = np.zeros(max_slots, dtype=np.int32)
        n = C.c_int()
        self.check(lib().pb_ctx_stamps_read(self.h, _p(st), _p(ids), C.c_int(max_slots), C.byref(n)))
        k = min(n.value, max_slots)
        return st[:k], ids[:k]

    def ep_probe_wait_timeout(self, spins: int = 2000):
        """Run one peer hand-shake whose partner never answers (pb_ep_probe_wait_timeout): raises PB_ERR_DEVICE once the
        bounded wait ran out; the context stays usable."""
        self.check(lib().pb_ep_probe_wait_timeout(self.h, C.c_uint(spins)))

    # ---- expert-parallel group (NCCL) ----
    def ep_unique_id(self) -> bytes:
        buf = C.create_string_buffer(128)
        self.check(lib().pb_ep_unique_id(self.h, buf))
        return buf.raw

    def ep_init(self, uid: bytes, rank: int, world: int):
        assert len(uid) == 128
        self.check(lib().pb_ep_init(self.h, C.c_char_p(uid), C.c_int(rank), C.c_int(world)))

    def close(self):
        if self.h:
            lib().pb_ctx_destroy(self.h)
            self.h = C.c_void_p()

    def kv4_pack(self, x: np.ndarray):
        x = _f32(x).reshape(-1)
        w = np.empty(x.size // 8, dtype=np.uint32)
        sc = np.empty(x.size // 32, dtype=np.float32)
        self.check(lib().pb_kv4_pack(self.h, _p(x), C.c_int64(x.size), _p(w), _p(sc)))
        return w, sc

    def kv4_unpack(self, w: np.ndarray, sc: np.ndarray, n: int):
        w = np.ascontiguousarray(w, dtype=np.uint32)
        sc = _f32(sc)
        x = np.empty(n, dtype=np.float32)
        self.check(lib().pb_kv4_unpack(self.h, _p(w), _p(sc), C.c_int64(n), _p(x)))
        return x


def type_geom(t: int):
    e, b = C.c_int(), C.c_int()
    if lib().pb_type_geom(C.c_int(t), C.byref(e), C.byref(b)):
        raise ValueError(f"unsupported ggml type {t}")
    return e.value, b.value


class QMat:
    """A quantized row-major matrix resident on the GPU in its native GGUF block format
    (QMat, src/model/gguf_q.rs:199-248)."""

    def __init__(self, ctx: Ctx, handle, t: int, rows: int, cols: int):
        self.ctx, self.h, self.ty, self.rows, self.cols = ctx, handle, t, rows, cols
        self.owned = True

    @classmethod
    def upload(cls, ctx: Ctx, t: int, rows: int, cols: int, raw: np.ndarray) -> "QMat":
        raw = np.ascontiguousarray(raw).view(np.uint8).reshape(-1)
        h = C.c_void_p()
        ctx.check(lib().pb_qmat_upload(ctx.h, C.c_int(t), C.c_int64(rows), C.c_int64(cols), _p(raw), C.c_size_t(raw.size), C.byref(h)))
        return cls(ctx, h, t, rows, cols)

    @classmethod
    def synth(cls, ctx: Ctx, t: int, rows: int, cols: int, seed: int, tid: int) -> "QMat":
        h = C.c_void_p()
        ctx.check(lib().pb_qmat_synth(ctx.h, C.c_int(t), C.c_int64(rows), C.c_int64(cols), C.c_uint64(seed), C.c_uint64(tid), C.byref(h)))
        return cls(ctx, h, t, rows, cols)

    @classmethod
    def synth_rows(cls, ctx: Ctx, t: int, rows: int, cols: int, seed: int, tid: int, row0: int) -> "QMat":
        """Rows [row0, row0 + rows) of the synthetic tensor (seed, tid)."""
        h = C.c_void_p()
        ctx.check(lib().pb_qmat_synth_rows(ctx.h, C.c_int(t), C.c_int64(rows), C.c_int64(cols), C.c_uint64(seed), C.c_uint64(tid), C.c_int64(row0), C.byref(h)))
        return cls(ctx, h, t, rows, cols)

    def row_bytes(self) -> int:
        e, b = type_geom(self.ty)
        return self.cols // e * b

    def nbytes(self) -> int:
        return self.rows * self.row_bytes()

    def raw_rows(self, r0: int, n: int) -> np.ndarray:
        out = np.empty(n * self.row_bytes(), dtype=np.uint8)
        self.ctx.check(lib().pb_qmat_read(self.ctx.h, self.h, C.c_int64(r0), C.c_int64(n), _p(out)))
        return out

    def to_f32(self, r0: int = 0, n: int | None = None) -> np.ndarray:
        n = self.rows - r0 if n is None else n
        out = np.empty((n, self.cols), dtype=np.float32)
        self.ctx.check(lib().pb_qmat_dequant(self.ctx.h, self.h, C.c_int64(r0), C.c_int64(n), _p(out)))
        return out

    def row(self, r: int) -> np.ndarray:
        return self.to_f32(r, 1)[0]

    def matmul(self, x: np.ndarray, t: int | None = None) -> np.ndarray:
        """y[t][rows] = x[t][cols] . W^T through the host-buffer entry point (QMat::matmul)."""
        x = _f32(x).reshape(-1, self.cols)
        t = x.shape[0] if t is None else t
        y = np.empty((t, self.rows), dtype=np.float32)
        self.ctx.check(lib().pb_gemv(self.ctx.h, self.h, _p(x), C.c_int(t), _p(y)))
        return y

    def matmul_static(self, x: np.ndarray, t: int | None = None) -> np.ndarray:
        """`matmul` without device allocation: stages through the fixed array built into the
        library (see pb_gemv_static); raises when t * (cols + rows) floats exceed that array."""
        x = _f32(x).reshape(-1, self.cols)
        t = x.shape[0] if t is None else t
        y = np.empty((t, self.rows), dtype=np.float32)
        self.ctx.check(lib().pb_gemv_static(self.ctx.h, self.h, _p(x), C.c_int(t), _p(y)))
        return y

    def matmul_dev(self, x_dev: int, t: int, y_dev: int):
        """Device-pointer form (pointers as integers, e.g. torch.Tensor.data_ptr())."""
        self.ctx.check(lib().pb_gemv_dev(self.ctx.h, self.h, C.c_void_p(x_dev), C.c_int(t), C.c_void_p(y_dev)))

    def free(self):
        if self.h and self.owned:
            lib().pb_qmat_free(self.h)
        self.h = C.c_void_p()
