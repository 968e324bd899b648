"""Checkpoint ingestion (SafeTensors -> .binfer, ainfer_binfer_from_safetensors) on the host.

A checkpoint is made from a seeded synthetic container by de-quantising every tensor and writing
the values out under Hugging Face names, in one file and as two shards with an index; the
converter must give back the container's directory and payloads byte for byte (the quantiser is
idempotent on de-quantised values: the group maximum is 7 scales, so scale and nibbles repeat),
the result must validate at the strictest level and decode the same tokens on the oracle. Then
the refusals: shapes that disagree with the architecture, a row length the quantiser cannot
group, an unknown dtype, offsets outside the file, a missing tensor."""
import json
import os
import struct

import numpy as np
import pytest

import oracle_lib as O
from test_host_cpu import _dir_entries


def _hf_name(n):
    n = n.replace("model.language_model.", "model.", 1) if n.startswith("model.language_model.") else n
    return n.replace(".mlp.shared.", ".mlp.shared_expert.")


def _entries(raw):
    out = {}
    for off, name in _dir_entries(raw):
        ndim = raw[off + 64]
        shape = list(struct.unpack_from("<8Q", raw, off + 72))[:ndim]
        storage = raw[off + 137]
        sc_off, sc_b, d_off, d_b = struct.unpack_from("<QQQQ", raw, off + 144)
        out[name] = dict(shape=shape, storage=storage, scales=bytes(raw[sc_off:sc_off + sc_b]), data=bytes(raw[d_off:d_off + d_b]))
    return out


def _dequant(e):
    if e["storage"] == 3:
        raw = np.frombuffer(e["data"], np.uint8)
        nib = np.empty(raw.size * 2, np.int8)
        nib[0::2] = raw & 0xF
        nib[1::2] = raw >> 4
        nib[nib >= 8] -= 16
        sc = O.bf16_to_f32(np.frombuffer(e["scales"], np.uint16))
        return (nib.astype(np.float32) * np.repeat(sc, 128)).reshape(e["shape"])
    return None


def _write_safetensors(path, tensors):
    """tensors: list of (name, dtype string, shape, raw bytes)."""
    header, blob = {}, bytearray()
    for name, dt, shape, raw in tensors:
        header[name] = {"dtype": dt, "shape": list(shape), "data_offsets": [len(blob), len(blob) + len(raw)]}
        blob += raw
    header["__metadata__"] = {"format": "pt"}
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj + bytes(blob))


@pytest.fixture(scope="module")
def checkpoint(tmp_path_factory):
    from ainfer_b200 import runtime
    d = tmp_path_factory.mktemp("ckpt")
    ref = str(d / "tiny.binfer")
    runtime.synth_write(ref, "tiny", seed=3)
    raw = open(ref, "rb").read()
    ents = _entries(raw)
    tensors = []
    for i, (name, e) in enumerate(sorted(ents.items())):
        if e["storage"] == 3:
            w = _dequant(e)
            if i % 3 == 0:
                tensors.append((_hf_name(name), "F16", e["shape"], w.astype(np.float16).tobytes()))   # exact: 4-bit x 8-bit values
            else:
                tensors.append((_hf_name(name), "F32", e["shape"], w.tobytes()))
        else:
            tensors.append((_hf_name(name), "BF16", e["shape"], e["data"]))
    tensors.append(("model.visual.blocks.0.attn.qkv.weight", "BF16", [4, 4], bytes(32)))   # vision tower: left out
    return dict(dir=d, ref=ref, raw=raw, ents=ents, tensors=tensors, arch=runtime.preset_config_json("tiny"))


def _same_as_reference(out, ck):
    from ainfer_b200 import runtime
    rc, msg = runtime.validate(out, 2)
    assert rc == 0, msg
    got = _entries(open(out, "rb").read())
    assert sorted(got) == sorted(ck["ents"]) and list(got) == sorted(got)   # same tensors; the converter writes them in name order
    for name, e in ck["ents"].items():
        assert got[name] == e, name


def test_single_file_round_trip(checkpoint):
    from ainfer_b200 import runtime
    src = str(checkpoint["dir"] / "model.safetensors")
    _write_safetensors(src, checkpoint["tensors"])
    out = str(checkpoint["dir"] / "single.binfer")
    runtime.from_safetensors(src, checkpoint["arch"], out)
    _same_as_reference(out, checkpoint)
    # the oracle decodes the same tokens from both containers
    a, b = O.Model(path=checkpoint["ref"]), O.Model(path=out)
    sa, sb = O.Session(a, 16), O.Session(b, 16)
    assert sa.decode_loop([5, 9, 2], 6)[0].tolist() == sb.decode_loop([5, 9, 2], 6)[0].tolist()
    sa.close(); sb.close(); a.close(); b.close()


def test_sharded_directory_round_trip(checkpoint):
    from ainfer_b200 import runtime
    d = checkpoint["dir"] / "sharded"
    d.mkdir()
    t = checkpoint["tensors"]
    half = len(t) // 2
    _write_safetensors(str(d / "model-00001-of-00002.safetensors"), t[:half])
    _write_safetensors(str(d / "model-00002-of-00002.safetensors"), t[half:])
    wm = {n: ("model-00001-of-00002.safetensors" if i < half else "model-00002-of-00002.safetensors")
          for i, (n, _, _, _) in enumerate(t)}
    (d / "model.safetensors.index.json").write_text(json.dumps({"metadata": {"total_size": 0}, "weight_map": wm}))
    out = str(checkpoint["dir"] / "sharded.binfer")
    runtime.from_safetensors(str(d), checkpoint["arch"], out)
    _same_as_reference(out, checkpoint)


def test_refusals(checkpoint, tmp_path):
    from ainfer_b200 import runtime
    t = checkpoint["tensors"]
    idx = {n: i for i, (n, _, _, _) in enumerate(t)}

    def attempt(tensors, name):
        src = str(tmp_path / f"{name}.safetensors")
        _write_safetensors(src, tensors)
        with pytest.raises(Exception) as e:
            runtime.from_safetensors(src, checkpoint["arch"], str(tmp_path / f"{name}.binfer"))
        assert not os.path.exists(str(tmp_path / f"{name}.binfer")) or os.path.getsize(str(tmp_path / f"{name}.binfer")) >= 0
        return str(e.value)

    # an expert matrix with half its rows: disagrees with the architecture
    bad = list(t)
    i = idx["model.layers.0.mlp.experts.3.gate_proj.weight"]
    n, dt, sh, raw = bad[i]
    bad[i] = (n, dt, [sh[0] // 2, sh[1]], raw[:len(raw) // 2])
    assert "unexpected shape of model.language_model.layers.0.mlp.experts.3.gate_proj.weight" in attempt(bad, "halfrows")
    # a tensor the runtime needs is missing
    bad = [x for x in t if x[0] != "model.layers.1.mlp.gate.weight"]
    assert "mlp.gate.weight" in attempt(bad, "missing")
    # a 2-D tensor whose rows the quantiser cannot group
    bad = list(t) + [("model.layers.0.extra.weight", "F32", [4, 100], bytes(1600))]
    assert "multiple of the quantiser's group of 128" in attempt(bad, "ragged")
    # unknown dtype
    bad = list(t) + [("model.layers.0.extra.count", "I64", [2], bytes(16))]
    assert "unsupported source dtype I64" in attempt(bad, "dtype")
    # payload shorter than the shape says
    n, dt, sh, raw = t[idx["lm_head.weight"]]
    bad = list(t)
    bad[idx["lm_head.weight"]] = (n, dt, sh, raw[:-4])
    assert "payload size does not match shape" in attempt(bad, "short")
    # offsets outside the file
    src = str(tmp_path / "trunc.safetensors")
    _write_safetensors(src, t)
    size = os.path.getsize(src)
    with open(src, "r+b") as f:
        f.truncate(size - 64)
    with pytest.raises(Exception) as e:
        runtime.from_safetensors(src, checkpoint["arch"], str(tmp_path / "trunc.binfer"))
    assert "outside the file" in str(e.value)
