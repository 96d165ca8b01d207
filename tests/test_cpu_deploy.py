"""The whole product as real processes without a GPU: ``xpool daemon serve`` + ``xpool ffnagent --backend cpu`` x 2 +
``xpool atnagent --backend cpu``; registration, placement, generation phases, handle brokering and readiness go
through the daemon; requests over HTTP; the answer must be the undivided model's; quiesce retires every agent."""
import os
import signal
import socket
import subprocess
import sys
import time
from pathlib import Path

import httpx
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _free_port_run(n: int, avoid: set[int]) -> int:
    """First of ``n`` consecutive free ports, none of them in ``avoid`` (attention device i listens on base + i)."""
    for _ in range(200):
        base = _free_port()
        if any(base + i in avoid for i in range(n)):
            continue
        held = []
        try:
            for i in range(n):
                sock = socket.socket()
                held.append(sock)
                sock.bind(("127.0.0.1", base + i))
            return base
        except OSError:
            continue
        finally:
            for sock in held:
                sock.close()
    raise RuntimeError("no run of free ports found")


def _toml(daemon_port: int, serve_port: int, models: str, atn=(0,), ffn=(1, 2), atn_extra="", serving_extra="") -> str:
    return f"""
[daemon]
port = {daemon_port}
[atn]
devices = {list(atn)}
{atn_extra}
[ffn]
devices = {list(ffn)}
[scheduler.slo]
ttft_ms = 2000
tbt_ms = 50
[serving]
base_port = {serve_port}
{serving_extra}
{models}
"""


plan_port = [0]          # the daemon port of the deployment a check callback is looking at


def _run(tmp_path, models_toml, check, atn=(0,), ffn=(1, 2), retire=True, atn_extra="", extra_env=None, before_ready=None,
         serving_extra=""):
    dport = _free_port()
    sport = _free_port_run(len(atn), {dport})
    plan_port[0] = dport
    cfgp = tmp_path / "xpool.toml"
    cfgp.write_text(_toml(dport, sport, models_toml, atn, ffn, atn_extra, serving_extra))
    env = dict(os.environ, XPOOL_CONFIG=str(cfgp), PYTHONPATH=str(ROOT), XPOOL_MAX_ROWS="128", XPOOL_MAX_BATCH="4",
               XPOOL_MAX_SEQ_LEN="128", **(extra_env or {}))
    xp = [sys.executable, "-m", "crosspool_b200.cli.main"]
    base = f"http://127.0.0.1:{dport}"
    procs = [subprocess.Popen(xp + ["daemon", "serve"], env=env)]
    try:
        for _ in range(150):
            try:
                if httpx.get(base + "/health", timeout=1).status_code == 200:
                    break
            except httpx.HTTPError:
                time.sleep(0.2)
        for role, dev in [("ffnagent", d) for d in ffn] + [("atnagent", d) for d in atn]:
            procs.append(subprocess.Popen(xp + [role, "--device", str(dev), "--backend", "cpu"], env=env))
        if before_ready is not None:
            before_ready(cfgp, base)
        ready = False
        for _ in range(400):
            r = httpx.get(base + "/ready", timeout=2).json()
            if r["system_ready"]:
                ready = True
                break
            assert r["failure"] is None, r
            assert all(p.poll() is None for p in procs), [p.poll() for p in procs]
            time.sleep(0.25)
        assert ready
        assert subprocess.run(xp + ["daemon", "check"], env=env, capture_output=True).returncode == 0
        if not retire:
            check(f"http://127.0.0.1:{sport}", base, procs)
            return
        check(f"http://127.0.0.1:{sport}", httpx.get(base + "/fabric/plan", timeout=2).json())
        assert httpx.post(base + "/fabric/quiesce", json={"reason": "test"}, timeout=5).status_code == 200
        for p in procs[1:]:
            assert p.wait(60) == 0
        assert httpx.get(base + "/fabric/plan", timeout=2).json()["phase"] == "stopped"
    finally:
        for p in procs:
            if p.poll() is None:
                p.send_signal(signal.SIGTERM)
        for p in procs:
            try:
                p.wait(10)
            except subprocess.TimeoutExpired:
                p.kill()
        # an agent that was killed cannot unlink its arenas: names carry this deployment's daemon port
        for f in Path("/dev/shm").glob(f"xp{dport}g*"):
            f.unlink(missing_ok=True)


def test_two_preset_models_on_a_shared_cpu_ffn_tier_answer_like_the_undivided_models(tmp_path):
    import zlib

    from crosspool_b200.models import config as mc
    from crosspool_b200.models.reference import ReferenceModel
    from crosspool_b200.models.weights import random_attention_weights, random_ffn_weights

    models = '[[models]]\nid = "tiny-qwen3"\nffn_tp_size = 2\n[[models]]\nid = "tiny-qwen3-moe"\nffn_tp_size = 2\n'

    def check(url, plan):
        assert {s["model_id"] for s in plan["shards"]} == {"tiny-qwen3", "tiny-qwen3-moe"}
        for mid in ("tiny-qwen3", "tiny-qwen3-moe"):
            prompt = list(range(3, 20))
            out = httpx.post(url + "/generate", json={"model": mid, "input_ids": prompt, "max_new_tokens": 5}, timeout=120).json()
            cfg, seed = mc.preset(mid), zlib.crc32(mid.encode()) % 1000
            whole = ReferenceModel(cfg, random_attention_weights(cfg, seed, dtype=torch.float32), random_ffn_weights(cfg, seed, dtype=torch.float32))
            want, _ = whole.generate(torch.tensor(prompt), 5)
            assert out["output_ids"] == want
        bad = httpx.post(url + "/generate", json={"model": "tiny-qwen3", "input_ids": [], "max_new_tokens": 5}, timeout=30)
        assert bad.status_code == 422                               # a malformed request is answered, the service goes on
        again = httpx.post(url + "/generate", json={"model": "tiny-qwen3", "input_ids": [5, 6, 7], "max_new_tokens": 2}, timeout=60)
        assert again.status_code == 200 and len(again.json()["output_ids"]) == 2
        # both processes answer a Prometheus scrape
        text = httpx.get(url + "/metrics", timeout=5).text
        assert 'xpool_requests_finished_total{model="tiny-qwen3"} 2' in text
        assert 'xpool_output_tokens_total{model="tiny-qwen3-moe"} 5' in text
        assert 'xpool_time_to_first_token_seconds_count{model="tiny-qwen3"} 2' in text and "xpool_engine_failed 0" in text
        dtext = httpx.get(url.rsplit(":", 1)[0] + f":{plan_port[0]}/metrics", timeout=5).text
        assert 'xpool_fabric_phase{phase="executable"} 1' in dtext and "xpool_system_ready 1" in dtext
        assert 'xpool_registered{role="ffnagent"} 2' in dtext

    _run(tmp_path, models, check)


def test_a_library_checkpoint_with_latent_attention_is_served_through_the_daemon(tmp_path):
    from crosspool_b200.devtools import hf_parity

    name = "DeepseekV2ForCausalLM/plain-q-yarn"
    if not hf_parity.available(name):
        pytest.skip("the installed transformers has no DeepseekV2")
    model = hf_parity.build_tiny_model(name)
    ckpt = tmp_path / "ckpt"
    model.save_pretrained(ckpt, safe_serialization=True)
    models = f'[[models]]\nid = "dsv2"\npath = "{ckpt}"\nffn_tp_size = 2\n'

    # the checkpoint ships a tokenizer: requests may carry text, answers carry the decoded text too
    from tokenizers import Tokenizer, pre_tokenizers
    from tokenizers import models as tok_models
    from transformers import PreTrainedTokenizerFast

    words = [f"w{i}" for i in range(1, 200)]
    wl = Tokenizer(tok_models.WordLevel({"<unk>": 0, **{w: i + 1 for i, w in enumerate(words)}}, unk_token="<unk>"))
    wl.pre_tokenizer = pre_tokenizers.Whitespace()
    PreTrainedTokenizerFast(tokenizer_object=wl, unk_token="<unk>").save_pretrained(ckpt)

    def check(url, plan):
        import json

        prompt = list(range(7, 21))
        out = httpx.post(url + "/generate", json={"input_ids": prompt, "max_new_tokens": 4}, timeout=120).json()
        with torch.no_grad():
            want = model.generate(torch.tensor([prompt]), max_new_tokens=4, do_sample=False)[0, len(prompt):].tolist()
        assert out["output_ids"] == want
        text = " ".join(f"w{i}" for i in prompt)             # word wN has id N
        by_text = httpx.post(url + "/generate", json={"text": text, "max_new_tokens": 4}, timeout=120).json()
        assert by_text["output_ids"] == want
        assert by_text["text"].split() == [f"w{i}" if 0 < i < 200 else "<unk>" for i in want]
        # streaming: one server-sent event per token, the last one marked finished
        with httpx.stream("POST", url + "/generate", json={"input_ids": prompt, "max_new_tokens": 4, "stream": True}, timeout=120) as r:
            events = [line[6:] for line in r.iter_lines() if line.startswith("data: ")]
        assert events[-1] == "[DONE]"
        toks = [json.loads(e) for e in events[:-1]]
        assert [t["token_id"] for t in toks] == want and [t["finished"] for t in toks] == [False, False, False, True]

    _run(tmp_path, models, check)


def test_data_parallel_attention_ranks_share_the_ffn_tier_behind_the_request_router(tmp_path):
    """One model as two data-parallel Instance ranks (two attention agents), FFN tensor-parallel over two FFN agents
    that keep one copy of the shard for both ranks; the request router spreads requests over the ranks by outstanding
    tokens and every answer is the undivided model's."""
    import asyncio
    import zlib

    from crosspool_b200.models import config as mc
    from crosspool_b200.models.reference import ReferenceModel
    from crosspool_b200.models.weights import random_attention_weights, random_ffn_weights
    from crosspool_b200.runtime.dp_router import DpRouter, create_router_app

    models = '[[models]]\nid = "tiny-qwen3"\natn_dp_size = 2\nffn_tp_size = 2\n'

    def check(url, plan):
        base = int(url.rsplit(":", 1)[1])
        ranks = [f"http://127.0.0.1:{base}", f"http://127.0.0.1:{base + 1}"]
        assert sorted((r["model_id"], r["rank"]) for r in plan["instance_ranks"]) == [("tiny-qwen3", 0), ("tiny-qwen3", 1)]
        router = DpRouter()
        for u in ranks:
            router.register("tiny-qwen3", u)
        app = create_router_app(router)
        cfg, seed = mc.preset("tiny-qwen3"), zlib.crc32(b"tiny-qwen3") % 1000
        whole = ReferenceModel(cfg, random_attention_weights(cfg, seed, dtype=torch.float32), random_ffn_weights(cfg, seed, dtype=torch.float32))
        prompts = [list(range(3 + i, 15 + 2 * i)) for i in range(4)]

        async def go():
            async with httpx.AsyncClient(transport=httpx.ASGITransport(app=app), base_url="http://router", timeout=120) as c:
                return await asyncio.gather(*[c.post("/generate", json={"model": "tiny-qwen3", "input_ids": p, "max_new_tokens": 4})
                                              for p in prompts])

        outs = asyncio.run(go())
        for p, r in zip(prompts, outs):
            assert r.status_code == 200
            assert r.json()["output_ids"] == whole.generate(torch.tensor(p), 4)[0]
        served = [b.served for b in router.backends["tiny-qwen3"]]
        assert sum(served) == 4 and min(served) >= 1              # both ranks took part
        # the same front end as a process that finds the ranks through the daemon (`xpool router`)
        rport = _free_port_run(1, {plan_port[0], base, base + 1})
        env = dict(os.environ, XPOOL_CONFIG=str(tmp_path / "xpool.toml"), PYTHONPATH=str(ROOT), XPOOL_MAX_ROWS="128", XPOOL_MAX_BATCH="4",
                   XPOOL_MAX_SEQ_LEN="128")
        proc = subprocess.Popen([sys.executable, "-m", "crosspool_b200.cli.main", "router", "--port", str(rport)], env=env)
        try:
            ranks_seen = {}
            for _ in range(100):
                try:
                    ranks_seen = httpx.get(f"http://127.0.0.1:{rport}/ranks", timeout=1).json()
                    if len(ranks_seen.get("tiny-qwen3", [])) == 2:
                        break
                except httpx.HTTPError:
                    pass
                time.sleep(0.2)
            assert sorted(b["url"] for b in ranks_seen["tiny-qwen3"]) == sorted(ranks)
            r = httpx.post(f"http://127.0.0.1:{rport}/generate", json={"model": "tiny-qwen3", "input_ids": prompts[0], "max_new_tokens": 4}, timeout=120)
            assert r.status_code == 200 and r.json()["output_ids"] == whole.generate(torch.tensor(prompts[0]), 4)[0]
        finally:
            proc.terminate()
            proc.wait(10)

    _run(tmp_path, models, check, atn=(0, 1), ffn=(2, 3))


def test_an_ffn_agent_that_dies_is_noticed_and_the_survivors_retire_the_generation(tmp_path):
    """Failure detection end to end, made on the host: an FFN agent process is killed between requests. The daemon's
    watchdog classifies the owner as exited and aborts the generation (fail-stop, no re-planning while serving);
    readiness reports the failure; the surviving agents quiesce, drain, finalise and exit cleanly."""
    models = '[[models]]\nid = "tiny-qwen3"\nffn_tp_size = 2\n'

    def check(url, base, procs):
        ok = httpx.post(url + "/generate", json={"input_ids": [4, 5, 6, 7], "max_new_tokens": 3}, timeout=120)
        assert ok.status_code == 200 and len(ok.json()["output_ids"]) == 3
        victim = procs[2]                                   # the second FFN agent
        victim.kill()
        victim.wait(10)
        failure = None
        for _ in range(120):
            r = httpx.get(base + "/ready", timeout=2).json()
            failure = r["failure"]
            if failure:
                break
            time.sleep(0.25)
        assert failure and "ffnagent:2" in failure and "exited" in failure, failure
        assert not r["system_ready"]
        for p in (procs[1], procs[3]):                      # the other FFN agent and the attention agent
            assert p.wait(60) == 0
        plan = httpx.get(base + "/fabric/plan", timeout=2).json()
        assert plan["phase"] == "stopped"
        with pytest.raises(httpx.HTTPError):                # the Instance no longer serves
            httpx.post(url + "/generate", json={"input_ids": [4, 5, 6], "max_new_tokens": 2}, timeout=5)

    _run(tmp_path, models, check, retire=False)


def test_elastic_kv_is_lent_from_an_idle_model_to_a_loaded_one_through_the_daemons_policy(tmp_path):
    """Two co-located models with elastic KV on a "device" of ten bundles: each starts with five. Four long requests
    for one model need seven; the engine publishes demand over the shared-memory channel, the daemon's policy shrinks
    the idle neighbour, then grows the borrower, the reconcilers carry the commands out, and every request is
    answered as the undivided model answers it."""
    import concurrent.futures as cf
    import zlib

    from crosspool_b200.models import config as mc
    from crosspool_b200.models.reference import ReferenceModel
    from crosspool_b200.models.weights import random_attention_weights, random_ffn_weights

    models = '[[models]]\nid = "tiny-qwen3"\nffn_tp_size = 2\n[[models]]\nid = "tiny-qwen3-moe"\nffn_tp_size = 2\n'
    bundle = 4 * (16 << 10)                     # 2 layers x (K, V) x 16 KiB

    def check(url, base, procs):
        st = {}
        for _ in range(100):                    # the policy freezes the pools once both partitions are described
            st = httpx.get(base + "/ecs/state", timeout=2).json()
            if st["frozen"] and all(p["mapped_bytes"] == 5 * bundle for p in st["partitions"]):
                break
            time.sleep(0.1)
        assert st["frozen"] and st["pools"]["0"]["budget_bytes"] == 10 * bundle
        assert sorted(p["target_bytes"] for p in st["partitions"]) == [5 * bundle, 5 * bundle]
        cfg, seed = mc.preset("tiny-qwen3"), zlib.crc32(b"tiny-qwen3") % 1000
        whole = ReferenceModel(cfg, random_attention_weights(cfg, seed, dtype=torch.float32), random_ffn_weights(cfg, seed, dtype=torch.float32))
        prompts = [[(7 * i + j) % 4000 + 1 for j in range(100)] for i in range(4)]      # 7 pages each: 28 pages = 7 bundles
        with cf.ThreadPoolExecutor(4) as pool:
            outs = list(pool.map(lambda p: httpx.post(url + "/generate", json={"model": "tiny-qwen3", "input_ids": p, "max_new_tokens": 6},
                                                      timeout=180).json(), prompts))
        for p, o in zip(prompts, outs):
            assert o["output_ids"] == whole.generate(torch.tensor(p), 6)[0]
        st = httpx.get(base + "/ecs/state", timeout=2).json()
        kinds = [(e["kind"], e["partition"]) for e in st["events"]]
        assert ("shrink", "tiny-qwen3-moe:0") in kinds and ("grow", "tiny-qwen3:0") in kinds
        assert kinds.index(("shrink", "tiny-qwen3-moe:0")) < kinds.index(("grow", "tiny-qwen3:0"))
        by = {p["key"]: p for p in st["partitions"]}
        assert by["tiny-qwen3:0"]["target_bytes"] >= 7 * bundle and by["tiny-qwen3-moe:0"]["target_bytes"] <= 3 * bundle
        assert sum(p["target_bytes"] for p in st["partitions"]) + st["pools"]["0"]["unassigned_bytes"] <= 10 * bundle
        # the lender still serves
        ok = httpx.post(url + "/generate", json={"model": "tiny-qwen3-moe", "input_ids": [3, 4, 5], "max_new_tokens": 2}, timeout=60)
        assert ok.status_code == 200
        assert httpx.post(base + "/fabric/quiesce", json={"reason": "test"}, timeout=5).status_code == 200
        for p in procs[1:]:
            assert p.wait(60) == 0

    _run(tmp_path, models, check, retire=False, atn_extra="elastic_kv = true\ndevice_memory_utilization = 1.0",
         extra_env={"XPOOL_CPU_KV_BYTES": str(10 * bundle)})


def test_a_library_model_joins_as_an_instance_rank_of_its_own_and_serves_through_the_brokered_arena(tmp_path):
    """The reference's process model on the CPU data plane: the engine (here the library model, in this test process)
    is an Instance rank of its own; the attention agent hosts nothing and only brokers the rank's arena; the rank
    registers, waits for the executable fabric, leases the arena from the daemon, maps the FFN ranks' arenas, detaches
    its FFNs, publishes *initialised*; then its own ``generate`` is served by the FFN agents. It leaves in order."""
    import threading

    from crosspool_b200 import config as C
    from crosspool_b200.devtools import hf_parity
    from crosspool_b200.integrations.transformers.instance import ExternalInstance

    name = "Qwen3MoeForCausalLM"
    if not hf_parity.available(name):
        pytest.skip(f"the installed transformers has no {name}")
    model = hf_parity.build_tiny_model(name)
    ckpt = tmp_path / "ckpt"
    model.save_pretrained(ckpt, safe_serialization=True)
    ids = torch.randint(0, model.config.vocab_size, (1, 9), generator=torch.Generator().manual_seed(3))
    with torch.no_grad():
        want = model.generate(ids, max_new_tokens=5, do_sample=False)
    models = f'[[models]]\nid = "acme/moe"\npath = "{ckpt}"\nffn_tp_size = 2\nexternal = true\n'
    box: dict = {}

    def before_ready(cfgp, base):
        # the rank joins while the agents come up: the daemon plans only once it has registered
        cfg = C.load_config(env={"XPOOL_CONFIG": str(cfgp), "XPOOL_MAX_ROWS": "128", "XPOOL_MAX_BATCH": "4", "XPOOL_MAX_SEQ_LEN": "128"})
        inst = ExternalInstance(cfg, "acme/moe", rank=0)
        box["inst"] = inst

        def join():
            try:
                box["report"] = inst.join(model)
            except Exception as e:       # surfaced by the assertions below
                box["error"] = e

        box["thread"] = threading.Thread(target=join)
        box["thread"].start()

    def check(url, base, procs):
        box["thread"].join(60)
        assert "error" not in box, box.get("error")
        inst = box["inst"]
        assert len(box["report"].shims) == model.config.num_hidden_layers and inst.runtime.state == "ready"
        insts = httpx.get(base + "/instances", timeout=2).json()
        assert "acme/moe" in str(insts)
        with pytest.raises(httpx.HTTPError):            # the attention agent hosts no engine for an external rank
            httpx.get(url + "/health", timeout=2)
        with torch.no_grad():
            got = model.generate(ids, max_new_tokens=5, do_sample=False)
        assert got.tolist() == want.tolist()
        assert inst.ffn_calls == 5 * model.config.num_hidden_layers
        assert inst.leave()
        assert httpx.post(base + "/fabric/quiesce", json={"reason": "test"}, timeout=5).status_code == 200
        for p in procs[1:]:
            assert p.wait(60) == 0

    _run(tmp_path, models, check, retire=False, before_ready=before_ready)


def test_an_engine_process_around_a_library_model_serves_requests_as_an_external_instance_rank(tmp_path):
    """Five processes: daemon, two FFN agents, the attention agent that brokers the arena, and an engine process of its
    own (``integrations.transformers.serve``) that loads an OPT checkpoint (LayerNorm, learned positions: an attention
    form the repository's GPU engine does not compute), joins as the model's Instance rank and answers over HTTP with
    the whole model's tokens. SIGTERM makes it leave in order."""
    from crosspool_b200.devtools import hf_parity

    name = "OPTForCausalLM"
    if not hf_parity.available(name):
        pytest.skip(f"the installed transformers has no {name}")
    model = hf_parity.build_tiny_model(name)
    ckpt = tmp_path / "ckpt"
    model.save_pretrained(ckpt, safe_serialization=True)
    models = f'[[models]]\nid = "acme/opt"\npath = "{ckpt}"\nffn_tp_size = 2\nexternal = true\n'
    box: dict = {}

    def before_ready(cfgp, base):
        import tomllib

        doc = tomllib.loads(cfgp.read_text())
        box["eport"] = _free_port_run(1, {doc["daemon"]["port"], doc["serving"]["base_port"]})
        env = dict(os.environ, XPOOL_CONFIG=str(cfgp), PYTHONPATH=str(ROOT), XPOOL_MAX_ROWS="128", XPOOL_MAX_BATCH="4",
                   XPOOL_MAX_SEQ_LEN="128")
        box["engine"] = subprocess.Popen([sys.executable, "-m", "crosspool_b200.integrations.transformers.serve", "--model-id", "acme/opt",
                                          "--port", str(box["eport"])], env=env, stderr=subprocess.PIPE, text=True)

    def check(url, base, procs):
        engine, eport = box["engine"], box["eport"]
        try:
            eurl = f"http://127.0.0.1:{eport}"
            for _ in range(200):
                try:
                    if httpx.get(eurl + "/health", timeout=1).status_code == 200:
                        break
                except httpx.HTTPError:
                    assert engine.poll() is None, engine.stderr.read()
                    time.sleep(0.25)
            inst = httpx.get(base + "/instances", timeout=2).json()
            assert str(eport) in str(inst)                               # the rank published its own serving listener
            prompt = list(range(5, 17))
            resp = httpx.post(eurl + "/generate", json={"input_ids": prompt, "max_new_tokens": 5}, timeout=120)
            assert resp.status_code == 200, resp.text
            out = resp.json()
            with torch.no_grad():
                want = model.generate(torch.tensor([prompt]), max_new_tokens=5, do_sample=False)[0, len(prompt):].tolist()
            assert out["output_ids"] == want
            assert httpx.get(eurl + "/health", timeout=2).json()["ffn_calls"] == 5 * model.config.num_hidden_layers
            assert httpx.post(eurl + "/generate", json={"input_ids": [], "max_new_tokens": 5}, timeout=10).status_code == 422
            engine.send_signal(signal.SIGTERM)
            assert engine.wait(30) == 0
            assert "left the deployment (clean)" in engine.stderr.read()
        finally:
            if engine.poll() is None:
                engine.kill()
        assert httpx.post(base + "/fabric/quiesce", json={"reason": "test"}, timeout=5).status_code == 200
        for p in procs[1:]:
            assert p.wait(60) == 0

    _run(tmp_path, models, check, retire=False, before_ready=before_ready)


def test_the_serving_engine_plugin_runs_its_whole_lifecycle_against_the_real_daemon_and_ffn_agents(tmp_path):
    """The plugin (hooks, adapter, lifecycle, shutdown) with a fake engine in this process, but nothing else faked:
    the daemon, the attention agent that brokers the arena and two FFN agents are real processes, the client is the real
    HTTP client, the FFN weights come from a checkpoint through the production loader. Loading the engine's model
    registers the Instance rank, waits for the executable fabric, leases the arena and binds the operator; a forward
    pass of the engine's own model then equals the same model with its FFNs computed locally from the checkpoint."""
    import types

    from safetensors.torch import save_file

    from crosspool_b200 import config as C
    from crosspool_b200.integrations.sglang import plugin, shim
    from crosspool_b200.integrations.transformers.attach import bind_cpu_tier
    from crosspool_b200.runtime.cpu_backends import attach_cpu_instance
    from crosspool_b200.runtime.instance import InstanceRankRuntime
    from crosspool_b200.service.client import XpoolClient
    from tests.sglang_fakes import PatchingHookRegistry, install_fake_engine

    hidden, inter, layers = 8, 16, 3
    ckpt = tmp_path / "ckpt"
    ckpt.mkdir()
    hf = {"architectures": ["Qwen3ForCausalLM"], "hidden_size": hidden, "num_hidden_layers": layers, "num_attention_heads": 4,
          "num_key_value_heads": 2, "head_dim": 2, "intermediate_size": inter, "vocab_size": 32, "hidden_act": "silu"}
    (ckpt / "config.json").write_text(__import__("json").dumps(hf))
    g = torch.Generator().manual_seed(11)
    tensors = {}
    for l in range(layers):
        for name, shape in (("gate_proj", (inter, hidden)), ("up_proj", (inter, hidden)), ("down_proj", (hidden, inter))):
            tensors[f"model.layers.{l}.mlp.{name}.weight"] = torch.randn(shape, generator=g) * 0.3
    save_file(tensors, str(ckpt / "model.safetensors"))
    models = f'[[models]]\nid = "acme/fake"\npath = "{ckpt}"\nffn_tp_size = 2\nexternal = true\n'
    box: dict = {}

    def before_ready(cfgp, base):
        import threading

        cfg = C.load_config(env={"XPOOL_CONFIG": str(cfgp), "XPOOL_MAX_ROWS": "128", "XPOOL_MAX_BATCH": "4", "XPOOL_MAX_SEQ_LEN": "128"})
        fake, reg = install_fake_engine(), PatchingHookRegistry()
        box.update(cfg=cfg, fake=fake, reg=reg)

        def runtime_factory(binding, rank, profile, device):
            def attach(arena, plan):
                t = attach_cpu_instance(cfg, plan, binding.model_id, rank)
                bind_cpu_tier(t.port)
                return t
            box["runtime"] = InstanceRankRuntime(XpoolClient(cfg.daemon_host, cfg.daemon_port), binding.model_id, rank, 0, profile, attach=attach)
            return box["runtime"]

        plugin.install(reg, environ={}, config=cfg, runtime_factory=runtime_factory)
        args = types.SimpleNamespace(model_path=str(ckpt), tp_size=1, dp_size=1, tp_rank=0, chunked_prefill_size=128, cuda_graph_max_bs=4,
                                     max_running_requests=4, cuda_graph_bs=[1, 2, 4], cuda_graph_backend_decode="full",
                                     cuda_graph_backend_prefill="breakable", host="127.0.0.1", port=30000)

        def boot():        # the engine starts: its scheduler constructs the model runner, which loads the model (hooked)
            try:
                box["sched"] = fake.sched.Scheduler(args)
                box["info"] = box["sched"].get_init_info()          # hooked: publishes initialised, waits for system ready
            except Exception as e:
                box["error"] = e

        box["thread"] = threading.Thread(target=boot)
        box["thread"].start()

    def check(url, base, procs):
        try:
            box["thread"].join(90)
            assert "error" not in box, repr(box.get("error"))
            sched, rt_ = box["sched"], box["runtime"]
            model = sched.model_runner.model
            assert [type(l.mlp).__name__ for l in model.model.layers] == ["FfnShimModule"] * layers and rt_.state == "ready"
            assert box["info"] == {"status": "ready"}
            inst = httpx.get(base + "/instances", timeout=2).json()["acme/fake:0"]
            assert inst["initialized"] and inst["max_prefill_rows"] == 128
            fb = types.SimpleNamespace(forward_mode=types.SimpleNamespace(name="DECODE"), dp_padding_mode=None)
            x = torch.randn(4, hidden, generator=g)
            with torch.no_grad():
                got = model(x, fb)
                want = x
                for l, layer in enumerate(model.model.layers):     # the same model with its FFNs computed here
                    want = want + layer.self_attn(want)
                    p = f"model.layers.{l}.mlp."
                    gate, up = want @ tensors[p + "gate_proj.weight"].t(), want @ tensors[p + "up_proj.weight"].t()
                    want = want + (torch.nn.functional.silu(gate) * up) @ tensors[p + "down_proj.weight"].t()
            torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-4)
            assert rt_.transport.port.calls == layers
            assert sched.run_event_loop() == "loop-done"
            assert sched.release_host_resources() == "released"     # ordered retirement through the plugin's shutdown hooks
            assert rt_.state == "detached"
            assert "acme/fake:0" not in httpx.get(base + "/instances", timeout=2).json()
        finally:
            box["reg"].restore()
            shim.bind_submit(None)
        assert httpx.post(base + "/fabric/quiesce", json={"reason": "test"}, timeout=5).status_code == 200
        for p in procs[1:]:
            assert p.wait(60) == 0

    _run(tmp_path, models, check, retire=False, before_ready=before_ready)


def test_an_external_ranks_elastic_kv_state_borrows_from_a_hosted_neighbour_through_the_daemon(tmp_path):
    """The plugin's elastic-KV state (what its hooks drive inside a serving engine) against the real control plane: an
    external Instance rank describes its partition in the daemon's channel next to a hosted model of the same device,
    its prefill is cut to the mapped backing, it publishes demand, the daemon shrinks the idle hosted neighbour and
    grows the external rank, and the same prefill then fits."""
    import threading

    from crosspool_b200 import config as C
    from crosspool_b200.ecs import reconciler as R
    from crosspool_b200.ecs import vmm
    from crosspool_b200.ecs.profile import KvPartitionGeometry
    from crosspool_b200.integrations.sglang.ecs_hooks import ElasticContextState
    from crosspool_b200.models import config as mc
    from crosspool_b200.native.runtime import EcsChannel
    from crosspool_b200.runtime.cpu_backends import attach_cpu_instance
    from crosspool_b200.runtime.instance import InstanceRankRuntime
    from crosspool_b200.service.client import XpoolClient
    from crosspool_b200.service.wire import InstanceFfnProfile

    models = ('[[models]]\nid = "tiny-qwen3"\nffn_tp_size = 2\n'
              '[[models]]\nid = "tiny-qwen3-moe"\nffn_tp_size = 2\nexternal = true\n')
    bundle = 4 * (16 << 10)
    box: dict = {}

    def before_ready(cfgp, base):
        cfg = C.load_config(env={"XPOOL_CONFIG": str(cfgp), "XPOOL_MAX_ROWS": "128", "XPOOL_MAX_BATCH": "4", "XPOOL_MAX_SEQ_LEN": "128"})
        client = XpoolClient(cfg.daemon_host, cfg.daemon_port)
        shape = mc.preset("tiny-qwen3-moe")
        rt_ = InstanceRankRuntime(client, "tiny-qwen3-moe", 0, 0, InstanceFfnProfile(max_prefill_rows=128, max_decode_rows=128,
                                                                                   hidden_size=shape.hidden_size),
                                  attach=lambda b, plan: attach_cpu_instance(cfg, plan, "tiny-qwen3-moe", 0))

        def boot():
            try:
                rt_.start()
                plan = rt_.wait_for_fabric_executable(timeout_s=90)
                rt_.attach_arena_from_daemon(plan)
                ref = None
                for _ in range(200):
                    try:
                        ref = client.ecs_channel(plan.generation)
                        break
                    except Exception:
                        time.sleep(0.05)
                ch = EcsChannel.attach(ref.name)
                cache = vmm.elastic_kv_cache(shape, 32, 16, "cpu", vmm.Driver.fake(1 << 40, granularity=16 << 10), None,
                                             initial_bundles=1, make_tensors=False, granularity=16 << 10)
                idx = ref.partitions["tiny-qwen3-moe:0"]
                KvPartitionGeometry.of(cache).describe(ch, idx, device=0, rank=0)
                box.update(state=ElasticContextState(cache, R.CapacityReconciler(cache, ch, idx), 16, ttft_slo_s=2.0), channel=ch, rt=rt_)
                rt_.publish_initialized(None)
                rt_.wait_for_ready(timeout_s=90)
            except Exception as e:
                box["error"] = e

        box["thread"] = threading.Thread(target=boot)
        box["thread"].start()

    def check(url, base, procs):
        box["thread"].join(120)
        assert "error" not in box, repr(box.get("error"))
        st = box["state"]
        for _ in range(100):                       # pools frozen, initial targets handed out and carried out on both sides
            st.begin_scheduling()
            view = httpx.get(base + "/ecs/state", timeout=2).json()
            if view["frozen"] and st.reconciler.mapped_bundles == 5:
                break
            time.sleep(0.1)
        # the agent reports the device's memory less what its own ranks hold; the policy adds every partition's floor back,
        # the external rank's included: one bundle more than the ten configured, left unassigned after the equal split
        assert st.reconciler.mapped_bundles == 5 and view["pools"]["0"]["budget_bytes"] == 11 * bundle
        want = 27 * 16                                                   # 28 pages with the next token: seven bundles
        cut = st.plan_prefill(seq_id=1, cached_tokens=0, want_tokens=want)
        assert cut.tokens == 20 * 16 and cut.missing_pages == 7 and st.stats["prefill_cut"] == 1
        st.finish_scheduling(cut.missing_pages, head_arrival_s=time.monotonic())
        fits = None
        for _ in range(100):
            st.begin_scheduling()
            fits = st.plan_prefill(seq_id=1, cached_tokens=0, want_tokens=want)
            if fits.tokens == want:
                break
            time.sleep(0.1)
        assert fits.tokens == want and st.reconciler.mapped_bundles == 7
        view = httpx.get(base + "/ecs/state", timeout=2).json()
        kinds = [(e["kind"], e["partition"]) for e in view["events"]]
        assert ("shrink", "tiny-qwen3:0") in kinds and ("grow", "tiny-qwen3-moe:0") in kinds
        # the hosted neighbour still serves while two of its bundles are on loan
        ok = httpx.post(url + "/generate", json={"model": "tiny-qwen3", "input_ids": [3, 4, 5], "max_new_tokens": 2}, timeout=60)
        assert ok.status_code == 200
        st.finish_scheduling(0)
        box["channel"].close()
        assert box["rt"].detach()
        assert httpx.post(base + "/fabric/quiesce", json={"reason": "test"}, timeout=5).status_code == 200
        for p in procs[1:]:
            assert p.wait(60) == 0

    _run(tmp_path, models, check, retire=False, before_ready=before_ready,
         atn_extra="elastic_kv = true\ndevice_memory_utilization = 1.0", extra_env={"XPOOL_CPU_KV_BYTES": str(10 * bundle)})


def test_the_benchmark_tool_brings_up_a_cpu_deployment_runs_a_case_and_its_result_is_reportable(tmp_path, capsys):
    """The serving benchmark end to end without a GPU: ``bench.serve_case`` starts the deployment as processes, drives
    the open-loop client of the smoke case against it (streaming requests, client-side TTFT / TPOT), retires it, and
    the suite runner's sealed result of the same runner is turned into a report."""
    import json

    from crosspool_b200.bench import report as R
    from crosspool_b200.bench import serve_case, suite

    dport = _free_port()
    sport = _free_port_run(1, {dport})
    out = tmp_path / "case.json"
    rc = serve_case.main(["--case", "smoke", "--models", "tiny-qwen3", "--atn", "0", "--ffn", "1", "2", "--ffn-tp", "2", "--backend", "cpu",
                          "--port", str(dport), "--serving-port", str(sport), "--max-batch", "4", "--max-seq-len", "128", "--max-rows", "128",
                          "--out", str(out)])
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rc == 0 and line["case"] == "smoke" and line["errors"] == 0 and line["completed"] > 0 and line["output_tok_per_s"] > 0
    doc = json.loads(out.read_text())
    assert doc["deployment"]["backend"] == "cpu" and doc["aggregate"]["tpot_ms"]["n"] > 0 and set(doc["per_model"]) == {"tiny-qwen3"}
    # the same result as a sealed suite repetition -> report
    run = tmp_path / "run"
    suite.run_suite([suite.CASES["smoke"]], {"tiny-qwen3": "unused"}, run, runner=lambda c, t, seed: doc)
    made = R.make_reports(run)
    assert (made[0] / "report.md").read_text().startswith("# smoke") and (made[0] / "throughput.svg").exists()


def test_attention_tensor_parallel_pair_serves_through_the_daemon_on_the_cpu_data_plane(tmp_path):
    """One Instance whose attention runs tensor-parallel over two attention agents (half of the heads each, output
    projections all-reduced, requests replicated from the first rank, which alone talks to the FFN tier and owns the
    HTTP endpoint); FFN tensor-parallel over two FFN agents. Answers equal the undivided model's."""
    import zlib

    from crosspool_b200.models import config as mc
    from crosspool_b200.models.reference import ReferenceModel
    from crosspool_b200.models.weights import random_attention_weights, random_ffn_weights

    rendezvous = _free_port_run(2, set())
    models = '[[models]]\nid = "tiny-qwen3"\natn_tp_size = 2\nffn_tp_size = 2\n'

    def check(url, plan):
        assert sorted((r["model_id"], r["rank"]) for r in plan["instance_ranks"]) == [("tiny-qwen3", 0), ("tiny-qwen3", 1)]
        cfg, seed = mc.preset("tiny-qwen3"), zlib.crc32(b"tiny-qwen3") % 1000
        whole = ReferenceModel(cfg, random_attention_weights(cfg, seed, dtype=torch.float32), random_ffn_weights(cfg, seed, dtype=torch.float32))
        for prompt in (list(range(3, 20)), [9, 8, 7, 6, 5]):
            out = httpx.post(url + "/generate", json={"input_ids": prompt, "max_new_tokens": 5}, timeout=120)
            assert out.status_code == 200, out.text
            assert out.json()["output_ids"] == whole.generate(torch.tensor(prompt), 5)[0]
        base = int(url.rsplit(":", 1)[1])
        with pytest.raises(httpx.HTTPError):                 # the second rank has no endpoint of its own
            httpx.get(f"http://127.0.0.1:{base + 1}/health", timeout=2)

    _run(tmp_path, models, check, atn=(0, 1), ffn=(2, 3), serving_extra=f"tp_rendezvous_base_port = {rendezvous}")


def test_tensor_parallel_ranks_agree_on_elastic_kv_growth_funded_by_their_neighbours(tmp_path):
    """A tensor-parallel Instance (one rank per attention device) next to a data-parallel co-tenant on each device, with
    elastic KV and four bundles per device. Long requests make both TP ranks publish demand; the daemon shrinks the idle
    co-tenant on each device and orders both ranks to grow; the ranks change capacity in the same engine step (they
    agree every poll over their gloo group), and the answers are the undivided model's."""
    import concurrent.futures as cf
    import zlib

    from crosspool_b200.models import config as mc
    from crosspool_b200.models.reference import ReferenceModel
    from crosspool_b200.models.weights import random_attention_weights, random_ffn_weights

    rendezvous = _free_port_run(2, set())
    models = ('[[models]]\nid = "tiny-qwen3"\natn_tp_size = 2\nffn_tp_size = 2\n'
              '[[models]]\nid = "tiny-qwen3-moe"\natn_dp_size = 2\nffn_tp_size = 2\n')
    bundle = 4 * (16 << 10)

    def check(url, base, procs):
        view = {}
        for _ in range(150):
            view = httpx.get(base + "/ecs/state", timeout=2).json()
            if view["frozen"] and all(p["mapped_bytes"] == p["target_bytes"] == 2 * bundle for p in view["partitions"]):
                break
            time.sleep(0.1)
        assert view["frozen"] and len(view["partitions"]) == 4, view
        cfg, seed = mc.preset("tiny-qwen3"), zlib.crc32(b"tiny-qwen3") % 1000
        whole = ReferenceModel(cfg, random_attention_weights(cfg, seed, dtype=torch.float32), random_ffn_weights(cfg, seed, dtype=torch.float32))
        prompts = [[(5 * i + j) % 4000 + 1 for j in range(100)] for i in range(3)]      # 7 pages each: 21 pages > the 16 mapped
        with cf.ThreadPoolExecutor(3) as pool:
            outs = list(pool.map(lambda p: httpx.post(url + "/generate", json={"model": "tiny-qwen3", "input_ids": p, "max_new_tokens": 5},
                                                      timeout=240).json(), prompts))
        for p, o in zip(prompts, outs):
            assert o["output_ids"] == whole.generate(torch.tensor(p), 5)[0]
        # the co-tenant's second data-parallel rank lives on the TP follower's device and answers there
        inst = httpx.get(base + "/instances", timeout=2).json()
        mcfg, mseed = mc.preset("tiny-qwen3-moe"), zlib.crc32(b"tiny-qwen3-moe") % 1000
        moe = ReferenceModel(mcfg, random_attention_weights(mcfg, mseed, dtype=torch.float32), random_ffn_weights(mcfg, mseed, dtype=torch.float32))
        for r in (0, 1):
            o = httpx.post(f"http://{inst[f'tiny-qwen3-moe:{r}']['listener']}/generate",
                           json={"model": "tiny-qwen3-moe", "input_ids": [3, 1, 4, 1, 5], "max_new_tokens": 4}, timeout=120).json()
            assert o["output_ids"] == moe.generate(torch.tensor([3, 1, 4, 1, 5]), 4)[0]
        assert inst["tiny-qwen3-moe:0"]["listener"] != inst["tiny-qwen3-moe:1"]["listener"]
        view = httpx.get(base + "/ecs/state", timeout=2).json()
        kinds = [(e["kind"], e["partition"]) for e in view["events"]]
        for r in (0, 1):
            assert ("shrink", f"tiny-qwen3-moe:{r}") in kinds and ("grow", f"tiny-qwen3:{r}") in kinds
        by = {p["key"]: p for p in view["partitions"]}
        assert by["tiny-qwen3:0"]["target_bytes"] == by["tiny-qwen3:1"]["target_bytes"] == 3 * bundle
        assert by["tiny-qwen3:0"]["mapped_bytes"] == by["tiny-qwen3:1"]["mapped_bytes"] == 3 * bundle      # grown together
        assert httpx.post(base + "/fabric/quiesce", json={"reason": "test"}, timeout=5).status_code == 200
        for p in procs[1:]:
            assert p.wait(90) == 0

    _run(tmp_path, models, check, atn=(0, 1), ffn=(2, 3), retire=False, atn_extra="elastic_kv = true\ndevice_memory_utilization = 1.0",
         serving_extra=f"tp_rendezvous_base_port = {rendezvous}", extra_env={"XPOOL_CPU_KV_BYTES": str(4 * bundle)})
