"""Serve recipe over a real socket: completions, chat, streaming, validation errors (CPU, random weights)."""

import http.client
import json
import threading

import pytest

from optimus_dl_b200.core import conf
from optimus_dl_b200.recipe.serve import ServeConfig, ServeRecipe


@pytest.fixture(scope="module")
def server():
    cfg = conf.merge(conf.create(ServeConfig()), conf.create({
        "serve": {"host": "127.0.0.1", "port": 0},
        "common": {"device": "cpu", "tokenizer": {"_name": "char_tokenize", "add_eos": False},
                   "model": {"_name": "llama2", "n_layer": 2, "n_head": 2, "n_embd": 32, "vocab_size": 258,
                             "sequence_length": 64, "intermediate_size": 64}},
    }))
    recipe = ServeRecipe(cfg)
    recipe.setup()
    httpd = recipe.make_server()
    t = threading.Thread(target=httpd.serve_forever, daemon=True)
    t.start()
    yield httpd.server_address[1]
    httpd.shutdown()
    httpd.server_close()


def _post(port, path, payload, raw=False):
    c = http.client.HTTPConnection("127.0.0.1", port, timeout=60)
    body = payload if isinstance(payload, (bytes, str)) else json.dumps(payload)
    c.request("POST", path, body=body, headers={"Content-Type": "application/json"})
    r = c.getresponse()
    data = r.read().decode("utf-8")
    c.close()
    return r.status, (data if raw else json.loads(data))


def test_completions(server):
    status, out = _post(server, "/v1/completions", {"prompt": "To be", "max_tokens": 8, "temperature": 0.0})
    assert status == 200 and out["object"] == "text_completion"
    assert out["usage"]["completion_tokens"] <= 8 and out["usage"]["prompt_tokens"] == 6  # BOS + 5 bytes
    status2, out2 = _post(server, "/v1/completions", {"prompt": "To be", "max_tokens": 8, "temperature": 0.0})
    assert out2["choices"][0]["text"] == out["choices"][0]["text"], "greedy decoding must repeat"


def test_chat_and_stream(server):
    msgs = [{"role": "user", "content": "hi"}]
    status, out = _post(server, "/v1/chat/completions", {"messages": msgs, "max_tokens": 5, "top_k": 5})
    assert status == 200 and out["choices"][0]["message"]["role"] == "assistant"
    status, raw = _post(server, "/v1/chat/completions", {"messages": msgs, "max_tokens": 5, "stream": True}, raw=True)
    assert status == 200
    events = [ln[6:] for ln in raw.split("\n") if ln.startswith("data: ")]
    assert events[-1] == "[DONE]"
    last = json.loads(events[-2])
    assert last["object"] == "chat.completion.chunk" and last["choices"][0]["finish_reason"] in ("stop", "length")


def test_long_prompt_is_cropped(server):
    status, out = _post(server, "/v1/completions", {"prompt": "x" * 500, "max_tokens": 4, "temperature": 0.0})
    assert status == 200 and out["usage"]["total_tokens"] <= 64


def test_errors(server):
    assert _post(server, "/v1/completions", "{not json")[0] == 400
    assert _post(server, "/v1/completions", {"max_tokens": 3})[0] == 422
    assert _post(server, "/v1/completions", {"prompt": "a", "max_tokens": 0})[0] == 422
    assert _post(server, "/nope", {})[0] == 404
    c = http.client.HTTPConnection("127.0.0.1", server, timeout=10)
    c.request("GET", "/health")
    assert c.getresponse().status == 200
