"""HTTP front end (ainfer_b200/server.py), protocol side, with a stub worker: endpoints, request
validation, completion object, server-sent-event framing, and that concurrent requests are served
one at a time (the reference's single-flight rule, tools/http/ainfer_http.py:39,136-137)."""
import json
import threading
import time
import urllib.error
import urllib.request

import pytest

from ainfer_b200 import server


class StubEngine:
    model_id, vocab = "stub", 100

    def __init__(self):
        self.active = self.max_active = 0

    def generate(self, ids, max_new, samp, on_token=None):
        self.active += 1
        self.max_active = max(self.max_active, self.active)
        gen = []
        for i in range(max_new):
            time.sleep(0.002)
            t = (sum(ids) + i + int(samp["seed"])) % self.vocab
            gen.append(t)
            if on_token:
                on_token(t)
        self.active -= 1
        return gen, 0.01


@pytest.fixture()
def srv():
    eng = StubEngine()
    s = server.serve(eng, server.IdTokenizer(eng.vocab), port=0)
    th = threading.Thread(target=s.serve_forever, daemon=True)
    th.start()
    yield f"http://127.0.0.1:{s.server_address[1]}", eng
    s.shutdown()


def _post(url, obj, raw=None):
    req = urllib.request.Request(url + "/v1/completions", data=raw if raw is not None else json.dumps(obj).encode(),
                                 headers={"Content-Type": "application/json"})
    try:
        with urllib.request.urlopen(req, timeout=30) as r:
            return r.status, r.read()
    except urllib.error.HTTPError as e:
        return e.code, e.read()


def test_endpoints_and_validation(srv):
    url, _ = srv
    assert json.load(urllib.request.urlopen(url + "/healthz")) == {"status": "ok"}
    assert json.load(urllib.request.urlopen(url + "/v1/models"))["data"][0]["id"] == "stub"
    assert _post(url, None, raw=b"{not json")[0] == 400
    assert _post(url, {"max_tokens": 3})[0] == 400                       # missing prompt
    assert _post(url, {"prompt": "1 2", "max_tokens": "x"})[0] == 400
    assert _post(url, {"prompt": "1 500"})[0] == 400                     # id outside the vocabulary
    code, body = _post(url, {"prompt": [1, 2, 3], "max_tokens": 4, "seed": 2})
    out = json.loads(body)
    assert code == 200 and out["choices"][0]["token_ids"] == [8, 9, 10, 11] and out["choices"][0]["text"] == "8 9 10 11"
    assert out["usage"] == {"prompt_tokens": 3, "completion_tokens": 4}
    code, body = _post(url, {"prompt": "4", "max_tokens": 100000})
    assert len(json.loads(body)["choices"][0]["token_ids"]) == server.MAX_NEW_LIMIT   # clamped like the reference's 512


def test_stream_framing(srv):
    url, _ = srv
    code, body = _post(url, {"prompt": "1 2 3", "max_tokens": 3, "stream": True})
    assert code == 200
    events = [e[len("data: "):] for e in body.decode().split("\n\n") if e]
    assert events[-1] == "[DONE]"
    chunks = [json.loads(e) for e in events[:-1]]
    assert [c["choices"][0]["token_ids"][0] for c in chunks[:-1]] == [6, 7, 8]
    assert chunks[-1]["choices"][0]["finish_reason"] == "stop"


def test_requests_are_served_one_at_a_time(srv):
    url, eng = srv
    th = [threading.Thread(target=_post, args=(url, {"prompt": "1", "max_tokens": 20})) for _ in range(4)]
    for t in th:
        t.start()
    for t in th:
        t.join()
    assert eng.max_active == 1
