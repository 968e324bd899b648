"""HTTP front end over the real worker (tiny synthetic model): a completion equals the session's
greedy tokens, streaming yields the same tokens one event each, sampling is reproducible by seed,
and a second request starts from a clean state."""
import json
import threading
import urllib.request

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _post(url, obj):
    req = urllib.request.Request(url + "/v1/completions", data=json.dumps(obj).encode(), headers={"Content-Type": "application/json"})
    with urllib.request.urlopen(req, timeout=120) as r:
        return r.read()


def test_completions_equal_the_session():
    from ainfer_b200 import runtime, server
    eng = server.Engine("synth:tiny:seed=1", max_ctx=128)
    srv = server.serve(eng, server.IdTokenizer(eng.vocab), port=0)
    th = threading.Thread(target=srv.serve_forever, daemon=True)
    th.start()
    url = f"http://127.0.0.1:{srv.server_address[1]}"
    prompt = [5, 17, 200 % eng.vocab, 9, 33]
    ref = runtime.Session(eng.model, 128)
    want = ref.generate(np.array(prompt, np.int32), 10).tolist()
    ref.close()
    for _ in range(2):                                # twice: the worker resets between requests
        out = json.loads(_post(url, {"prompt": prompt, "max_tokens": 10}))
        assert out["choices"][0]["token_ids"] == want
    events = [e[len("data: "):] for e in _post(url, {"prompt": " ".join(map(str, prompt)), "max_tokens": 10, "stream": True}).decode().split("\n\n") if e]
    assert events[-1] == "[DONE]"
    assert [json.loads(e)["choices"][0]["token_ids"][0] for e in events[:-2]] == want
    a = json.loads(_post(url, {"prompt": prompt, "max_tokens": 12, "temperature": 0.9, "top_k": 20, "top_p": 0.95, "seed": 7, "rep_penalty": 1.1}))
    b = json.loads(_post(url, {"prompt": prompt, "max_tokens": 12, "temperature": 0.9, "top_k": 20, "top_p": 0.95, "seed": 7, "rep_penalty": 1.1}))
    c = json.loads(_post(url, {"prompt": prompt, "max_tokens": 12, "temperature": 0.9, "top_k": 20, "top_p": 0.95, "seed": 8, "rep_penalty": 1.1}))
    assert a["choices"][0]["token_ids"] == b["choices"][0]["token_ids"]
    assert a["choices"][0]["token_ids"] != c["choices"][0]["token_ids"] or a["choices"][0]["token_ids"] != want
    srv.shutdown()
    eng.close()
