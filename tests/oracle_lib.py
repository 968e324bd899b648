"""ctypes binding of the CPU oracle (oracle/_build/liboracle.so).

Test infrastructure: imported by tests, the smoke check and the bench's CPU
baseline only. Builds the library with oracle/Makefile on first use.
"""
import ctypes as C
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
LIB_PATH = os.path.join(ORACLE_DIR, "_build", "liboracle.so")

_lib = None

f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
i8p = np.ctypeslib.ndpointer(np.int8, flags="C_CONTIGUOUS")
u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
u16p = np.ctypeslib.ndpointer(np.uint16, flags="C_CONTIGUOUS")
i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")


def build(force=False):
    srcs = [os.path.join(ORACLE_DIR, f) for f in ("oracle.cpp", "oracle_ops.h", "oracle_math.h")]
    stale = (not os.path.exists(LIB_PATH)) or any(
        os.path.getmtime(s) > os.path.getmtime(LIB_PATH) for s in srcs)
    if force or stale:
        subprocess.run(["make", "-C", ORACLE_DIR], check=True, stdout=subprocess.DEVNULL)
    return LIB_PATH


def lib():
    global _lib
    if _lib is not None:
        return _lib
    build()
    L = C.CDLL(LIB_PATH)
    vp, i, f, u64, d = C.c_void_p, C.c_int, C.c_float, C.c_uint64, C.c_double
    sig = {
        "orc_model_open": (vp, [C.c_char_p, i, C.c_char_p, i]),
        "orc_model_new": (vp, [C.c_char_p]),
        "orc_model_synth": (vp, [C.c_char_p, u64]),
        "orc_model_add_tensor": (None, [vp, C.c_char_p, i, i, C.POINTER(u64), vp, u64, vp, u64]),
        "orc_model_close": (None, [vp]),
        "orc_model_arch_json": (C.c_char_p, [vp]),
        "orc_model_tensor_count": (i, [vp]),
        "orc_model_tensor_info": (i, [vp, C.c_char_p, C.POINTER(i), C.POINTER(i), C.POINTER(u64),
                                      C.POINTER(vp), C.POINTER(u64), C.POINTER(vp), C.POINTER(u64)]),
        "orc_session_new": (vp, [vp, i]),
        "orc_session_free": (None, [vp]),
        "orc_session_buf": (vp, [vp, i, C.POINTER(u64)]),
        "orc_step": (i, [vp, i, i, i]),
        "orc_mtp_step": (i, [vp, i, i, f32p, f32p]),
        "orc_decode_loop": (d, [vp, i32p, i, i, i, i32p]),
        "orc_moe_block": (None, [vp, C.c_char_p, f32p, f32p, i32p, f32p]),
        "orc_threads": (i, []),
        "orc_quantize_int4": (None, [f32p, u64, u8p, u16p]),
        "orc_aquant": (None, [f32p, i, i8p, f32p]),
        "orc_gemv_a8": (None, [u8p, u16p, i, i, i8p, f32p, f32p]),
        "orc_gemv_a16": (None, [u8p, u16p, i, i, f32p, i, f32p]),
        "orc_rmsnorm": (None, [f32p, f32p, i, f, f32p]),
        "orc_headnorm": (None, [f32p, f32p, i, f, f32p]),
        "orc_rope_table": (None, [i, i, d, f32p, f32p]),
        "orc_rope_apply": (None, [f32p, i, f32p, f32p]),
        "orc_kv_quant_row": (None, [f32p, i, i8p, u16p]),
        "orc_attn_bf16kv": (None, [f32p, u16p, u16p, f32p, i, i, i, i, f32p, vp]),
        "orc_attn_int8kv": (None, [f32p, i8p, u16p, i8p, u16p, f32p, i, i, i, i, f32p]),
        "orc_conv_silu": (None, [f32p, f32p, f32p, i, f32p]),
        "orc_l2norm": (None, [f32p, i, f, f32p]),
        "orc_dn_beta": (f, [f]),
        "orc_dn_gdecay": (f, [f, f, f]),
        "orc_deltanet_head": (None, [f32p, f32p, f32p, f32p, f, f, i, f32p]),
        "orc_gated_norm": (None, [f32p, f32p, f32p, i, f32p]),
        "orc_dot_bf16": (f, [u16p, f32p, i]),
        "orc_router_topk": (None, [f32p, i, i, i32p, f32p, C.POINTER(f)]),
        "orc_argmax": (i, [f32p, i]),
        "orc_expf": (f, [f]),
        "orc_logf": (f, [f]),
        "orc_f32_to_f16": (C.c_uint16, [f]),
        "orc_f16_to_f32": (f, [C.c_uint16]),
        "orc_f32_to_bf16": (C.c_uint16, [f]),
        "orc_crc32": (C.c_uint32, [u8p, u64]),
        "orc_synth_normal": (None, [C.c_char_p, u64, u64, u64, f, f32p]),
        "orc_draw_u32": (C.c_uint32, [C.c_char_p, u64, u64]),
        "orc_normal_from_u32": (f, [C.c_uint32]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args
    _lib = L
    return L


# ------------------------------------------------------------ numpy helpers ---
def bf16_bits(a):
    """fp32 -> BF16 bits, round to nearest even (same rule as the oracle)."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    return ((u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)


def bf16_to_f32(b):
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def quantize_int4(w):
    """w: fp32 [N, K] -> (packed u8 [N, K/2], scales u16 [N, K/128])."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    n = w.size
    packed = np.zeros(((n + 127) // 128) * 64, np.uint8)
    scales = np.zeros((n + 127) // 128, np.uint16)
    lib().orc_quantize_int4(w.reshape(-1), n, packed, scales)
    if w.ndim == 2 and w.shape[1] % 128 == 0:
        return packed.reshape(w.shape[0], w.shape[1] // 2), scales.reshape(w.shape[0], w.shape[1] // 128)
    return packed, scales


def aquant(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    q = np.zeros(x.size, np.int8)
    s = np.zeros(x.size // 128, np.float32)
    lib().orc_aquant(x, x.size, q, s)
    return q, s


def gemv_a8(P, S, xq, sq):
    N, K = P.shape[0], P.shape[1] * 2
    y = np.zeros(N, np.float32)
    lib().orc_gemv_a8(np.ascontiguousarray(P), np.ascontiguousarray(S), N, K, xq, sq, y)
    return y


def gemv_a16(P, S, x):
    """x: fp32 [M, K] holding bf16-representable values -> y [M, N]."""
    N, K = P.shape[0], P.shape[1] * 2
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, K)
    y = np.zeros((x.shape[0], N), np.float32)
    lib().orc_gemv_a16(np.ascontiguousarray(P), np.ascontiguousarray(S), N, K, x, x.shape[0], y)
    return y


def synth_normal(name, seed, count, std, first=0):
    out = np.zeros(count, np.float32)
    lib().orc_synth_normal(name.encode(), seed, first, count, std, out)
    return out


class Model:
    def __init__(self, path=None, arch_json=None, check_crc=True, synth_seed=None):
        L = lib()
        self._keep = []
        if synth_seed is not None:
            self.h = L.orc_model_synth(arch_json.encode(), synth_seed)
        elif path is not None:
            err = C.create_string_buffer(512)
            self.h = L.orc_model_open(os.fsencode(path), int(check_crc), err, 512)
            if not self.h:
                raise ValueError(err.value.decode())
        else:
            self.h = L.orc_model_new(arch_json.encode())

    def add_tensor(self, name, storage, shape, data, scales=None):
        sh = (C.c_uint64 * 8)(*list(shape))
        self._keep.append((data, scales))
        lib().orc_model_add_tensor(
            self.h, name.encode(), storage, len(shape), sh,
            data.ctypes.data, data.nbytes,
            scales.ctypes.data if scales is not None else None,
            scales.nbytes if scales is not None else 0)

    @property
    def arch_json(self):
        return lib().orc_model_arch_json(self.h).decode()

    def tensor(self, name):
        st, nd = C.c_int(), C.c_int()
        shape = (C.c_uint64 * 8)()
        dp, sp = C.c_void_p(), C.c_void_p()
        db, sb = C.c_uint64(), C.c_uint64()
        r = lib().orc_model_tensor_info(self.h, name.encode(), C.byref(st), C.byref(nd), shape,
                                        C.byref(dp), C.byref(db), C.byref(sp), C.byref(sb))
        if r != 0:
            raise KeyError(name)
        data = np.ctypeslib.as_array((C.c_uint8 * db.value).from_address(dp.value)) if db.value else None
        scales = (np.ctypeslib.as_array((C.c_uint16 * (sb.value // 2)).from_address(sp.value))
                  if sb.value else None)
        return dict(storage=st.value, shape=list(shape)[:nd.value], data=data, scales=scales)

    def close(self):
        if self.h:
            lib().orc_model_close(self.h)
            self.h = None


class Session:
    BUFS = dict(conv=(0, np.float32), S=(1, np.float32), Kc=(2, np.int8), Vc=(3, np.int8),
                Ks=(4, np.uint16), Vs=(5, np.uint16), logits=(6, np.float32), routed=(7, np.int32),
                near_gap=(8, np.float32), layer_out=(9, np.float32), hidden=(10, np.float32))

    def __init__(self, model, max_ctx):
        self.model = model
        self.h = lib().orc_session_new(model.h, max_ctx)

    def buf(self, name):
        which, dt = self.BUFS[name]
        n = C.c_uint64()
        p = lib().orc_session_buf(self.h, which, C.byref(n))
        if n.value == 0:
            return np.zeros(0, dt)
        raw = (C.c_uint8 * n.value).from_address(p)
        return np.frombuffer(raw, dtype=dt)

    def step(self, token, pos, want_logits=True):
        return lib().orc_step(self.h, token, pos, int(want_logits))

    def decode_loop(self, prompt, n_gen, start_pos=0):
        prompt = np.ascontiguousarray(prompt, dtype=np.int32)
        out = np.zeros(max(n_gen, 1), np.int32)
        secs = lib().orc_decode_loop(self.h, prompt, len(prompt), n_gen, start_pos, out)
        return out[:n_gen], secs

    def close(self):
        if self.h:
            lib().orc_session_free(self.h)
            self.h = None


def preset_json(name):
    """Architecture JSON of a named synthetic shape (oracle/presets.json; the same shapes as the
    runtime's presets, which a test compares)."""
    import json
    with open(os.path.join(ORACLE_DIR, "presets.json")) as f:
        return json.dumps(json.load(f)[name], separators=(",", ":"))


def model_from_device(dev, model):
    """Oracle model whose tensors are host copies of a device model's two weight arenas.
    dev: ainfer_b200.cuda_abi.Device, model: ainfer_b200.runtime.Model (both passed in: this
    module never imports the product)."""
    n = model.tensor_count()
    infos = [model.tensor_at(i) for i in range(n)]
    spans = {}
    for kind, ptr_of, len_of in (("data", lambda t: t.data, lambda t: t.data_bytes),
                                 ("scales", lambda t: t.scales, lambda t: t.scale_bytes)):
        live = [(ptr_of(t), len_of(t)) for t in infos if len_of(t)]
        lo = min(p for p, _ in live)
        hi = max(p + b for p, b in live)
        host = np.empty(hi - lo, np.uint8)
        step = 1 << 30
        for off in range(0, hi - lo, step):
            nb = min(step, hi - lo - off)
            host[off:off + nb] = dev.download(lo + off, nb, np.uint8)
        spans[kind] = (lo, host)
    om = Model(arch_json=model.config_json)
    for t in infos:
        lo, host = spans["data"]
        data = host[t.data - lo:t.data - lo + t.data_bytes]
        scales = None
        if t.scale_bytes:
            slo, shost = spans["scales"]
            scales = shost[t.scales - slo:t.scales - slo + t.scale_bytes].view(np.uint16)
        om.add_tensor(t.name.decode(), t.storage, list(t.shape)[:t.ndim], data, scales)
    return om
