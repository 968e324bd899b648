"""ctypes binding of the decode runtime C ABI (include/ainfer_runtime.h)."""
import ctypes as C
import os

import numpy as np

from . import cuda_abi

RUNTIME_LIB = os.path.join(cuda_abi.LIB_DIR, "libainfer_runtime.so")
DECODE_EXE = os.path.join(cuda_abi.LIB_DIR, "ainfer_decode")

_vp, _i, _u64 = C.c_void_p, C.c_int, C.c_uint64
_pp = C.POINTER(C.c_void_p)


class TensorInfo(C.Structure):
    _fields_ = [("name", C.c_char * 64), ("storage", C.c_int32), ("ndim", C.c_int32),
                ("shape", C.c_uint64 * 8), ("data", C.c_void_p), ("data_bytes", C.c_uint64),
                ("scales", C.c_void_p), ("scale_bytes", C.c_uint64)]


class SampleParams(C.Structure):
    _fields_ = [("temp", C.c_float), ("top_k", C.c_int32), ("top_p", C.c_float),
                ("rep_penalty", C.c_float), ("seed", C.c_uint64)]


SIGNATURES = {
    "ainfer_rt_last_error": (C.c_char_p, []),
    "ainfer_binfer_validate": (_i, [C.c_char_p, _i]),
    "ainfer_synth_write": (_i, [C.c_char_p, C.c_char_p, _u64]),
    "ainfer_preset_config_json": (C.c_char_p, [C.c_char_p]),
    "ainfer_binfer_from_safetensors": (_i, [C.c_char_p, C.c_char_p, C.c_char_p]),
    "ainfer_model_open": (_i, [_vp, C.c_char_p, _i, _pp]),
    "ainfer_model_close": (_i, [_vp]),
    "ainfer_model_config_json": (C.c_char_p, [_vp]),
    "ainfer_model_tensor_count": (_i, [_vp]),
    "ainfer_model_tensor_at": (_i, [_vp, _i, C.POINTER(TensorInfo)]),
    "ainfer_model_tensor": (_i, [_vp, C.c_char_p, C.POINTER(TensorInfo)]),
    "ainfer_model_bytes": (_i, [_vp, C.POINTER(_u64), C.POINTER(_u64)]),
    "ainfer_session_create": (_i, [_vp, _i, _i, _pp]),
    "ainfer_session_destroy": (_i, [_vp]),
    "ainfer_session_reset": (_i, [_vp]),
    "ainfer_session_buffer": (_i, [_vp, C.c_char_p, _pp, C.POINTER(_u64)]),
    "ainfer_session_step": (_i, [_vp, _i, _i, C.POINTER(_i)]),
    "ainfer_session_prefill": (_i, [_vp, C.POINTER(_i), _i, _i]),
    "ainfer_session_prefill_ep": (_i, [_vp, C.c_char_p, _i, _i]),
    "ainfer_session_prefill_rows": (_i, [_vp, _i]),
    "ainfer_session_generate": (_i, [_vp, C.POINTER(_i), _i, _i, _i, C.POINTER(_i), C.POINTER(C.c_float)]),
    "ainfer_session_logits": (_i, [_vp, _vp]),
    "ainfer_session_sample": (_i, [_vp, C.POINTER(SampleParams), _vp, _i, C.POINTER(_u64), C.POINTER(_i)]),
    "ainfer_session_launches_per_token": (_i, [_vp, C.POINTER(_u64)]),
    "ainfer_session_mtp_draft": (_i, [_vp, _i, _i, _i, C.POINTER(_i)]),
    "ainfer_session_mtp_logits": (_i, [_vp, _vp]),
    "ainfer_session_generate_mtp": (_i, [_vp, _vp, _i, _i, _i, _i, _vp, _vp]),
    "ainfer_ep_unique_id": (_i, [_vp]),
    "ainfer_ep_create": (_i, [_vp, _vp, _i, _i, _i, _i, C.POINTER(_vp)]),
    "ainfer_ep_destroy": (_i, [_vp]),
    "ainfer_ep_buffer": (_i, [_vp, C.c_char_p, C.POINTER(_vp), C.POINTER(C.c_uint64)]),
    "ainfer_ep_moe_layer": (_i, [_vp, _i]),
    "ainfer_ep_moe_stack": (_i, [_vp, _i, _i, _vp]),
    "ainfer_batch_create": (_i, [_vp, _vp, _i, _i, _i, _i, _i, C.POINTER(_vp)]),
    "ainfer_batch_destroy": (_i, [_vp]),
    "ainfer_batch_buffer": (_i, [_vp, C.c_char_p, C.POINTER(_vp), C.POINTER(C.c_uint64)]),
    "ainfer_batch_step": (_i, [_vp]),
    "ainfer_apply_rep_penalty": (_i, [_vp, _i, _vp, _i, C.c_float]),
    "ainfer_sample_token": (_i, [_vp, _i, C.POINTER(SampleParams), C.POINTER(_u64), _vp]),
}

_lib = None


class RuntimeError_(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"ainfer runtime rc={code}: {msg}")
        self.code = code


def load():
    global _lib
    if _lib is None:
        cuda_abi.load()
        if not os.path.exists(RUNTIME_LIB):
            raise ImportError(f"{RUNTIME_LIB} is missing: build it with `python -m ainfer_b200._build`")
        L = C.CDLL(RUNTIME_LIB, mode=C.RTLD_GLOBAL)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


def _check(rc):
    if rc:
        raise RuntimeError_(rc, (load().ainfer_rt_last_error() or b"").decode())


def synth_write(path, preset, seed=0):
    _check(load().ainfer_synth_write(os.fsencode(path), preset.encode(), seed))


def validate(path, level=2):
    """Returns (rc, message)."""
    L = load()
    rc = L.ainfer_binfer_validate(os.fsencode(path), level)
    return rc, ((L.ainfer_rt_last_error() or b"").decode() if rc else "")


def preset_config_json(preset):
    r = load().ainfer_preset_config_json(preset.encode())
    return r.decode() if r else None


class Model:
    def __init__(self, dev, spec, validate_level=1):
        self.dev = dev
        h = C.c_void_p()
        _check(load().ainfer_model_open(dev.h, os.fsencode(spec), validate_level, C.byref(h)))
        self.h = h

    @property
    def config_json(self):
        return load().ainfer_model_config_json(self.h).decode()

    @property
    def config(self):
        import json
        return json.loads(self.config_json)

    def tensor_count(self):
        return load().ainfer_model_tensor_count(self.h)

    def tensor_at(self, i):
        info = TensorInfo()
        _check(load().ainfer_model_tensor_at(self.h, i, C.byref(info)))
        return info

    def tensor(self, name):
        info = TensorInfo()
        _check(load().ainfer_model_tensor(self.h, name.encode(), C.byref(info)))
        return info

    def nbytes(self):
        a, b = C.c_uint64(), C.c_uint64()
        _check(load().ainfer_model_bytes(self.h, C.byref(a), C.byref(b)))
        return a.value, b.value

    def close(self):
        if self.h:
            load().ainfer_model_close(self.h)
            self.h = None


class Session:
    DIAG = 1
    PER_LAYER_LISTS = 2
    MULTI_KERNEL = 4
    STAGE_CLOCK = 8
    PERSISTENT = 16

    def __init__(self, model, max_ctx, flags=0):
        self.model = model
        self.dev = model.dev
        h = C.c_void_p()
        _check(load().ainfer_session_create(model.h, max_ctx, flags, C.byref(h)))
        self.h = h
        self.max_ctx = max_ctx

    def buffer(self, which):
        p, n = C.c_void_p(), C.c_uint64()
        _check(load().ainfer_session_buffer(self.h, which.encode(), C.byref(p), C.byref(n)))
        return p.value, n.value

    def read(self, which, dtype):
        p, n = self.buffer(which)
        return self.dev.download(p, n // np.dtype(dtype).itemsize, dtype)

    def write(self, which, arr):
        p, n = self.buffer(which)
        arr = np.ascontiguousarray(arr)
        assert arr.nbytes == n, (which, arr.nbytes, n)
        self.dev.write(p, arr)

    def reset(self):
        _check(load().ainfer_session_reset(self.h))

    def step(self, token, pos):
        out = C.c_int()
        _check(load().ainfer_session_step(self.h, token, pos, C.byref(out)))
        return out.value

    def generate(self, prompt, n_gen, start_pos=0, timed=False):
        prompt = np.ascontiguousarray(prompt, dtype=np.int32)
        out = np.zeros(max(n_gen, 1), np.int32)
        ms = C.c_float()
        _check(load().ainfer_session_generate(
            self.h, prompt.ctypes.data_as(C.POINTER(C.c_int)), len(prompt), n_gen, start_pos,
            out.ctypes.data_as(C.POINTER(C.c_int)), C.byref(ms) if timed else None))
        return (out[:n_gen], ms.value) if timed else out[:n_gen]

    def logits(self):
        V = self.model.config["vocab"]
        out = np.zeros(V, np.float32)
        _check(load().ainfer_session_logits(self.h, out.ctypes.data))
        return out

    def sample(self, temp, top_k=0, top_p=1.0, rep_penalty=1.0, seen=(), rng=1):
        """Samples from the last step's logits on the device. Returns (token, new rng state)."""
        p = SampleParams(temp, top_k, top_p, rep_penalty, 0)
        seen = np.ascontiguousarray(seen, np.int32)
        state, tok = C.c_uint64(rng), C.c_int()
        _check(load().ainfer_session_sample(self.h, C.byref(p), seen.ctypes.data if seen.size else None, seen.size,
                                            C.byref(state), C.byref(tok)))
        return tok.value, state.value

    def prefill(self, tokens, start_pos=0):
        """Advances the state over the tokens in passes of up to 192 rows (no logits)."""
        t = np.ascontiguousarray(tokens, np.int32)
        _check(load().ainfer_session_prefill(self.h, t.ctypes.data_as(C.POINTER(C.c_int)), len(t), int(start_pos)))

    def prefill_rows(self, rows):
        """Rows per pass of the next prefill (rows x world x top-k <= 2048; default the largest multiple of 8 within that, at most 192)."""
        _check(load().ainfer_session_prefill_rows(self.h, int(rows)))

    def prefill_ep(self, rank, world, nccl_id=None):
        """Expert parallelism for this session's prefill: every rank prefills its own sequence of the
        same length, passes of up to 2048 / (top-k x world) rows; nccl_id = ep_unique_id() of one rank."""
        _check(load().ainfer_session_prefill_ep(self.h, nccl_id, int(rank), int(world)))

    def mtp_draft(self, next_token, pos, from_trunk=True):
        """One draft of the MTP head (hidden input: the trunk's last residual, or chained)."""
        d = _i()
        _check(load().ainfer_session_mtp_draft(self.h, int(next_token), int(pos), 1 if from_trunk else 0, C.byref(d)))
        return d.value

    def mtp_logits(self):
        out = np.zeros(self.model.config["vocab"], np.float32)
        _check(load().ainfer_session_mtp_logits(self.h, out.ctypes.data))
        return out

    def generate_mtp(self, prompt, n_gen, draft_k=3, start_pos=0):
        """Greedy generation with draft_k MTP drafts per round. Returns (tokens, {rounds, drafted, accepted})."""
        prompt = np.ascontiguousarray(prompt, dtype=np.int32)
        out = np.zeros(n_gen, np.int32)
        st = np.zeros(3, np.int32)
        _check(load().ainfer_session_generate_mtp(self.h, prompt.ctypes.data, len(prompt), n_gen, start_pos, draft_k,
                                                  out.ctypes.data, st.ctypes.data))
        return out, {"rounds": int(st[0]), "drafted": int(st[1]), "accepted": int(st[2])}

    def launches_per_token(self):
        n = C.c_uint64()
        _check(load().ainfer_session_launches_per_token(self.h, C.byref(n)))
        return n.value

    def close(self):
        if self.h:
            load().ainfer_session_destroy(self.h)
            self.h = None


def sample_token(logits, temp=0.0, top_k=0, top_p=1.0, rep_penalty=1.0, seed=0, rng=None, want_probs=False):
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    p = SampleParams(temp, top_k, top_p, rep_penalty, seed)
    state = C.c_uint64(seed if rng is None else rng)
    probs = np.zeros(logits.size, np.float32) if want_probs else None
    tok = load().ainfer_sample_token(logits.ctypes.data, logits.size, C.byref(p), C.byref(state),
                                     probs.ctypes.data if want_probs else None)
    return tok, state.value, probs


def apply_rep_penalty(logits, seen, penalty):
    logits = np.ascontiguousarray(logits, dtype=np.float32).copy()
    seen = np.ascontiguousarray(seen, dtype=np.int32)
    load().ainfer_apply_rep_penalty(logits.ctypes.data, logits.size, seen.ctypes.data, seen.size, penalty)
    return logits


def from_safetensors(src, arch_json, out_path):
    """SafeTensors file or sharded directory -> .binfer (ainfer_binfer_from_safetensors)."""
    _check(load().ainfer_binfer_from_safetensors(str(src).encode(), arch_json.encode(), str(out_path).encode()))


def ep_unique_id():
    """128 bytes of a fresh NCCL id (one rank calls it and hands the bytes to the others)."""
    buf = C.create_string_buffer(128)
    _check(load().ainfer_ep_unique_id(buf))
    return buf.raw


class EpMoe:
    """Expert-parallel MoE block of a loaded model for a decode batch (ainfer_ep_*): this rank
    owns batch/world rows and experts/world experts. world == 1 needs no NCCL id."""
    ROUTER_BIAS = 1

    def __init__(self, model, batch, rank=0, world=1, nccl_id=None, flags=0):
        self.model, self.dev = model, model.dev
        self.batch, self.rank, self.world = batch, rank, world
        h = C.c_void_p()
        idb = C.create_string_buffer(nccl_id, 128) if nccl_id is not None else None
        _check(load().ainfer_ep_create(model.h, idb, rank, world, batch, flags, C.byref(h)))
        self.h = h
        cfg = model.config
        self.rows, self.hidden, self.top_k = batch // world, cfg["hidden"], cfg["top_k"]

    def buffer(self, which):
        p, n = C.c_void_p(), C.c_uint64()
        _check(load().ainfer_ep_buffer(self.h, which.encode(), C.byref(p), C.byref(n)))
        return p.value, n.value

    def read(self, which, dtype):
        p, n = self.buffer(which)
        return self.dev.download(p, n // np.dtype(dtype).itemsize, dtype)

    def write(self, which, arr):
        p, n = self.buffer(which)
        arr = np.ascontiguousarray(arr)
        assert arr.nbytes == n, (which, arr.nbytes, n)
        self.dev.write(p, arr)

    def layer(self, layer, res):
        """x = res + MoE(norm(res)) for this rank's rows [rows][H] (blocking)."""
        self.write("res", np.asarray(res, np.float32))
        _check(load().ainfer_ep_moe_layer(self.h, int(layer)))
        self.dev.sync()
        return self.read("x", np.float32).reshape(self.rows, self.hidden)

    def stack(self, first, count, segments=False):
        """`count` layers from `first`, chained through the "res" buffer; asynchronous unless
        segments is set (then returns the summed ms of the five segments)."""
        seg = (C.c_float * 5)() if segments else None
        _check(load().ainfer_ep_moe_stack(self.h, int(first), int(count), seg))
        return list(seg) if segments else None

    def close(self):
        if self.h:
            load().ainfer_ep_destroy(self.h)
            self.h = None


class BatchDecode:
    """Batched decode (ainfer_batch_*): this rank owns batch/world sequences; every step advances
    each of them by one greedy token on the device."""
    ROUTER_BIAS = 1

    def __init__(self, model, batch, max_ctx, rank=0, world=1, nccl_id=None, flags=0):
        self.model, self.dev = model, model.dev
        h = C.c_void_p()
        idb = C.create_string_buffer(nccl_id, 128) if nccl_id is not None else None
        _check(load().ainfer_batch_create(model.h, idb, rank, world, batch, max_ctx, flags, C.byref(h)))
        self.h, self.rows = h, batch // world

    def buffer(self, which):
        p, n = C.c_void_p(), C.c_uint64()
        _check(load().ainfer_batch_buffer(self.h, which.encode(), C.byref(p), C.byref(n)))
        return p.value, n.value

    def read(self, which, dtype):
        p, n = self.buffer(which)
        return self.dev.download(p, n // np.dtype(dtype).itemsize, dtype)

    def write(self, which, arr):
        p, n = self.buffer(which)
        arr = np.ascontiguousarray(arr)
        assert arr.nbytes == n, (which, arr.nbytes, n)
        self.dev.write(p, arr)

    def set_inputs(self, tokens, positions):
        """Control block of every owned sequence: the token to feed and its position."""
        c = np.zeros((self.rows, 4), np.int32)
        c[:, 0], c[:, 1], c[:, 2], c[:, 3] = tokens, positions, np.asarray(positions) + 1, -1
        self.write("ctrl", c)

    def step(self):
        _check(load().ainfer_batch_step(self.h))

    def tokens(self):
        self.dev.sync()
        return self.read("out_tok", np.int32)

    def close(self):
        if self.h:
            load().ainfer_batch_destroy(self.h)
            self.h = None
