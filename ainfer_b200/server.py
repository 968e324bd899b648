"""OpenAI-style HTTP front end over a PERSISTENT in-process worker.

Endpoints and request fields of the reference's daemon (tools/http/ainfer_http.py:89-183):
  GET  /healthz        -> {"status": "ok"}
  GET  /v1/models      -> {"data": [{"id": <model>, ...}]}
  POST /v1/completions -> {prompt, max_tokens, temperature, top_k, top_p, seed, rep_penalty, stream}
    stream=false: one completion object; stream=true: server-sent events, one `data:` chunk per
    generated token, then `data: [DONE]`.
The reference spawns its decode binary for every request and pays the model load each time (it
names a persistent worker as follow-on work, :14-15); here the model is loaded once and one session
serves all requests behind a single-flight lock (the device decodes one sequence at a time). The
prompt goes through the chunked prefill, generated tokens through the persistent decode step;
with temperature > 0 the device sampler picks the token (the reference's sampler semantics; the
logits stay on the device).

Without tokenizer assets a prompt is a list of token ids (or a string of ids separated by spaces)
and the completion text is the generated ids separated by spaces; with `--tokenizer tokenizer.json`
(Hugging Face `tokenizers` format) text goes in and out.

Usage: python -m ainfer_b200.server --model model.binfer|synth:<preset> [--port 8010] [--max-ctx 8192]
"""
import argparse
import json
import threading
import time
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer

import numpy as np

MAX_NEW_LIMIT = 512


class IdTokenizer:
    """Stand-in when no tokenizer assets are given: text is token ids separated by spaces."""

    def __init__(self, vocab):
        self.vocab = vocab

    def encode(self, prompt):
        if isinstance(prompt, list) and all(isinstance(t, int) for t in prompt):
            ids = prompt
        elif isinstance(prompt, str):
            ids = [int(t) for t in prompt.split()]
        else:
            raise ValueError("prompt must be a list of token ids or a string of ids")
        if not ids or any(t < 0 or t >= self.vocab for t in ids):
            raise ValueError("token id out of range")
        return ids

    def decode(self, ids):
        return " ".join(str(int(t)) for t in ids)


class HfTokenizer:
    def __init__(self, path):
        from tokenizers import Tokenizer
        self.t = Tokenizer.from_file(path)

    def encode(self, prompt):
        if isinstance(prompt, list):
            prompt = " ".join(map(str, prompt))
        ids = self.t.encode(prompt).ids
        if not ids:
            raise ValueError("empty prompt")
        return ids

    def decode(self, ids):
        return self.t.decode([int(t) for t in ids])


class Engine:
    """The persistent worker: one model, one session, one request at a time."""

    def __init__(self, spec, max_ctx=8192, device=0):
        from . import cuda_abi, runtime
        self.runtime = runtime
        self.dev = cuda_abi.Device(device)
        self.model = runtime.Model(self.dev, spec)
        self.vocab = self.model.config["vocab"]
        self.max_ctx = max_ctx
        self.sess = runtime.Session(self.model, max_ctx, runtime.Session.PERSISTENT)
        self.model_id = spec.split("/")[-1]

    def generate(self, ids, max_new, samp, on_token=None):
        """ids: prompt token ids. Returns (generated ids, wall seconds)."""
        rt, s = self.runtime, self.sess
        if len(ids) + max_new + 8 > self.max_ctx:
            raise ValueError(f"prompt of {len(ids)} tokens + {max_new} new exceed the context of {self.max_ctx}")
        t0 = time.time()
        s.reset()
        ids = np.asarray(ids, np.int32)
        P = len(ids)
        if P > 1:
            s.prefill(ids[:-1])
        gen, tok, pos = [], int(ids[-1]), P - 1
        sampling = samp.get("temperature", 0) > 0
        rng = int(samp.get("seed", 0)) or 0x9E3779B97F4A7C15
        seen = [int(t) for t in ids]
        for _ in range(max_new):
            nxt = s.step(tok, pos)                      # greedy token; logits stay on the device
            if sampling:                                # on the device: 12 bytes come back, not the logits
                nxt, rng = s.sample(float(samp["temperature"]), int(samp.get("top_k", 0)), float(samp.get("top_p", 1.0)),
                                    float(samp.get("rep_penalty", 1.0)), seen, rng)
            gen.append(int(nxt))
            seen.append(int(nxt))
            if on_token:
                on_token(int(nxt))
            tok, pos = int(nxt), pos + 1
        return gen, time.time() - t0

    def close(self):
        self.sess.close(); self.model.close(); self.dev.close()


def make_handler(engine, tokenizer, lock):
    class Handler(BaseHTTPRequestHandler):
        server_version = "ainfer-b200/1.0"

        def _send(self, code, obj):
            body = json.dumps(obj).encode()
            self.send_response(code)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(body)))
            self.end_headers()
            self.wfile.write(body)

        def log_message(self, *a):
            pass

        def do_GET(self):
            if self.path == "/healthz":
                self._send(200, {"status": "ok"})
            elif self.path == "/v1/models":
                self._send(200, {"data": [{"id": engine.model_id, "owned_by": "ainfer"}]})
            else:
                self._send(404, {"error": "not found"})

        def do_POST(self):
            if self.path != "/v1/completions":
                self._send(404, {"error": "not found"})
                return
            try:
                n = int(self.headers.get("Content-Length", 0))
                body = json.loads(self.rfile.read(n) or b"{}")
                if not isinstance(body, dict):
                    raise ValueError
            except Exception:
                self._send(400, {"error": "invalid JSON"})
                return
            prompt = body.get("prompt", "")
            if not prompt:
                self._send(400, {"error": "missing prompt"})
                return
            try:
                max_new = int(body.get("max_tokens", 16))
            except Exception:
                self._send(400, {"error": "bad max_tokens"})
                return
            max_new = max(1, min(max_new, MAX_NEW_LIMIT))
            try:
                samp = {"temperature": float(body.get("temperature", 0) or 0), "top_k": int(body.get("top_k", 0) or 0),
                        "top_p": float(body.get("top_p", 1.0) or 1.0), "seed": int(body.get("seed", 0) or 0),
                        "rep_penalty": float(body.get("rep_penalty", 1.0) or 1.0)}
            except Exception:
                self._send(400, {"error": "bad sampling parameter"})
                return
            try:
                ids = tokenizer.encode(prompt)
            except Exception as e:
                self._send(400, {"error": f"tokenize failed: {e}"})
                return
            if body.get("stream"):
                self._stream(ids, max_new, samp)
            else:
                self._complete(ids, max_new, samp)

        def _complete(self, ids, max_new, samp):
            try:
                with lock:
                    gen, wall = engine.generate(ids, max_new, samp)
            except ValueError as e:
                self._send(400, {"error": str(e)})
                return
            except Exception as e:
                self._send(500, {"error": str(e)})
                return
            self._send(200, {"id": "ainfer-0", "model": engine.model_id,
                             "choices": [{"text": tokenizer.decode(gen), "index": 0, "finish_reason": "stop", "token_ids": gen}],
                             "usage": {"prompt_tokens": len(ids), "completion_tokens": len(gen)},
                             "timings": {"wall_s": round(wall, 3)}})

        def _stream(self, ids, max_new, samp):
            self.send_response(200)
            self.send_header("Content-Type", "text/event-stream")
            self.send_header("Cache-Control", "no-cache")
            self.end_headers()

            def emit(obj):
                self.wfile.write(f"data: {json.dumps(obj)}\n\n".encode())
                self.wfile.flush()

            try:
                with lock:
                    engine.generate(ids, max_new, samp, on_token=lambda t: emit(
                        {"id": "ainfer-0", "model": engine.model_id,
                         "choices": [{"text": tokenizer.decode([t]), "index": 0, "finish_reason": None, "token_ids": [t]}]}))
                emit({"id": "ainfer-0", "model": engine.model_id, "choices": [{"text": "", "index": 0, "finish_reason": "stop"}]})
                self.wfile.write(b"data: [DONE]\n\n")
                self.wfile.flush()
            except BrokenPipeError:
                pass
            except Exception as e:
                try:
                    emit({"error": str(e)})
                except BrokenPipeError:
                    pass

    return Handler


def serve(engine, tokenizer, port=8010, host="127.0.0.1"):
    """Returns the server (call serve_forever(), or run it in a thread; shutdown() stops it)."""
    return ThreadingHTTPServer((host, port), make_handler(engine, tokenizer, threading.Lock()))


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True, help=".binfer path or synth:<preset>[:seed=N]")
    ap.add_argument("--port", type=int, default=8010)
    ap.add_argument("--max-ctx", type=int, default=8192)
    ap.add_argument("--tokenizer", default=None, help="tokenizer.json (Hugging Face tokenizers); default: token ids as text")
    args = ap.parse_args(argv)
    engine = Engine(args.model, args.max_ctx)
    tok = HfTokenizer(args.tokenizer) if args.tokenizer else IdTokenizer(engine.vocab)
    srv = serve(engine, tok, args.port)
    print(f"serving {engine.model_id} on 127.0.0.1:{args.port}", flush=True)
    try:
        srv.serve_forever()
    finally:
        engine.close()


if __name__ == "__main__":
    main()
