"""Least-outstanding-tokens routing over a model's Instance ranks, with fake rank endpoints."""
import json

import httpx
import pytest
from fastapi.testclient import TestClient

from crosspool_b200.runtime.dp_router import DpRouter, create_router_app


def test_pick_prefers_the_least_loaded_healthy_rank():
    r = DpRouter()
    for u in ("http://a", "http://b", "http://a"):
        r.register("m", u)
    assert len(r.backends["m"]) == 2
    a = r.pick("m", 1000)
    b = r.pick("m", 10)
    c = r.pick("m", 10)
    assert (a.url, b.url, c.url) == ("http://a", "http://b", "http://b")
    r.done(b, 10)
    r.done(a, 1000, ok=False)          # a failed: taken out of rotation
    assert r.pick("m", 5).url == "http://b"
    with pytest.raises(LookupError):
        r.pick("other", 1)


def test_router_app_relays_plain_and_streaming_requests():
    seen = []

    def handler(request: httpx.Request) -> httpx.Response:
        body = json.loads(request.content)
        seen.append((request.url.host, body["max_new_tokens"]))
        if body.get("stream"):
            return httpx.Response(200, content=b'data: {"token_id": 1, "index": 1, "finished": true}\n\ndata: [DONE]\n\n',
                                  headers={"content-type": "text/event-stream"})
        return httpx.Response(200, json={"output_ids": [7] * body["max_new_tokens"], "rank": request.url.host})

    router = DpRouter()
    router.register("m", "http://rank0")
    router.register("m", "http://rank1")
    app = create_router_app(router, transport=httpx.MockTransport(handler))
    with TestClient(app) as c:
        outs = [c.post("/generate", json={"model": "m", "input_ids": [1] * n, "max_new_tokens": 2}).json()["rank"]
                for n in (100, 5, 5)]
        assert outs == ["rank0", "rank1", "rank0"]          # requests complete at once, so served counts break the tie
        s = c.post("/generate", json={"model": "m", "input_ids": [1], "max_new_tokens": 1, "stream": True})
        assert s.status_code == 200 and "[DONE]" in s.text
        snap = c.get("/ranks").json()["m"]
        assert sum(b["served"] for b in snap) == 4 and all(b["inflight"] == 0 and b["outstanding_tokens"] == 0 for b in snap)
        assert c.post("/generate", json={"model": "zzz", "input_ids": [1]}).status_code == 503


def test_ranks_are_discovered_from_the_daemons_listing_and_vanished_ones_stop_receiving_requests():
    import types

    from crosspool_b200.runtime.dp_router import DpRouter, discover_ranks

    table = {"m/a:0": {"initialized": True, "listener": "127.0.0.1:30000"}, "m/a:1": {"initialized": True, "listener": "127.0.0.1:30001"},
             "m/a:2": {"initialized": False, "listener": "127.0.0.1:30002"},             # still warming up
             "m/b:0": {"initialized": True, "listener": None},                            # hosted, no listener of its own
             "m/c:0": {"initialized": True, "listener": "127.0.0.1:30100"}}
    http = types.SimpleNamespace(get=lambda url, timeout: types.SimpleNamespace(json=lambda: table))
    r = DpRouter()
    assert discover_ranks(r, "http://daemon", ["m/a"], http=http) == 2
    assert [b.url for b in r.backends["m/a"]] == ["http://127.0.0.1:30000", "http://127.0.0.1:30001"] and "m/c" not in r.backends
    del table["m/a:1"]                                                   # the rank left (or its agent died)
    table["m/a:2"]["initialized"] = True
    assert discover_ranks(r, "http://daemon", ["m/a"], http=http) == 2
    health = {b.url: b.healthy for b in r.backends["m/a"]}
    assert health == {"http://127.0.0.1:30000": True, "http://127.0.0.1:30001": False, "http://127.0.0.1:30002": True}
    assert r.pick("m/a", 10).url != "http://127.0.0.1:30001" and r.pick("m/a", 10).url != "http://127.0.0.1:30001"
    assert discover_ranks(r, "http://daemon", None, http=http) == 3 and "m/c" in r.backends
