"""The user documentation embeds tables that the code prints; they must not drift apart."""

import re
from pathlib import Path

DOCS = Path(__file__).resolve().parents[1] / "docs"


def _generated(page: str) -> str:
    text = (DOCS / page).read_text()
    m = re.search(r"<!-- generated: [^>]* -->\n(.*?)<!-- end generated -->", text, re.S)
    assert m, f"{page} has no generated block"
    return m.group(1)


def test_configuration_page_lists_exactly_the_registry():
    from crosspool_b200 import config as C

    assert _generated("configuration.md") == C.reference_markdown()
    assert all(s.description for s in C.CONFIG_REGISTRY)


def test_supported_models_page_is_what_the_adapters_and_engines_implement():
    from crosspool_b200.models import adapters
    from crosspool_b200.models.support import support_markdown, supported_architectures

    assert _generated("supported-models.md") == support_markdown()
    rows = {r.architecture: r for r in supported_architectures()}
    assert set(rows) == set(adapters.ADAPTERS)
    assert rows["Qwen3ForCausalLM"].gpu_attention and not rows["DeepseekV2ForCausalLM"].gpu_attention
    assert all(r.engine_adapter for r in rows.values())


def test_every_page_of_the_index_exists_and_commands_named_in_the_docs_parse():
    index = (DOCS / "README.md").read_text()
    for page in re.findall(r"\]\(([\w\-]+\.md)\)", index):
        assert (DOCS / page).exists(), page
    from crosspool_b200.cli.main import _parser

    p = _parser()
    for argv in (["config", "dump"], ["config", "reference"], ["config", "models"], ["daemon", "check"], ["daemon", "serve"],
                 ["atnagent", "--device", "0"], ["ffnagent", "--device", "1"], ["memory-profile", "--calibrate", "--out", "p.json"]):
        p.parse_args(argv)


def test_cli_prints_the_generated_tables(capsys):
    from crosspool_b200.cli.main import main

    assert main(["config", "reference"]) == 0
    assert "`scheduler.ffn_policy`" in capsys.readouterr().out
    assert main(["config", "models"]) == 0
    assert "`GptOssForCausalLM`" in capsys.readouterr().out


def test_every_variable_of_the_example_environment_file_is_one_the_code_reads():
    from crosspool_b200 import config as C

    root = DOCS.parent
    names = set(re.findall(r"^#?\s*([A-Z][A-Z0-9_]+)=", (root / ".env.example").read_text(), re.M))
    known = {s.env_var for s in C.CONFIG_REGISTRY if s.env_var} | {"XPOOL_NVTX", "XPOOL_CPU_KV_BYTES", "SGLANG_PLUGINS"}
    assert names <= known, names - known
    assert (root / "configs" / "xpool.example.toml").exists()


def test_http_api_page_lists_exactly_the_routes_the_apps_serve():
    from crosspool_b200 import config as C
    from crosspool_b200.runtime.serving import create_serving_app
    from crosspool_b200.service.daemon.app import create_app
    from crosspool_b200.service.daemon.control import ControlPlane

    text = (DOCS / "http-api.md").read_text()
    instance_part, daemon_part = text.split("## Daemon")
    rows = lambda part: {(m, p.replace("{model_id}", "{model_id:path}")) for m, p in re.findall(r"^\| (GET|POST) \| `([^`]+)` \|", part, re.M)}
    builtin = {"/openapi.json", "/docs", "/docs/oauth2-redirect", "/redoc"}
    served = lambda app: {(m, r.path) for r in app.routes if hasattr(r, "methods") and r.path not in builtin for m in r.methods
                          if m in ("GET", "POST")}
    cfg = C.load_config(toml_text="[atn]\ndevices=[0]\n[ffn]\ndevices=[1]\n[scheduler.slo]\nttft_ms=1\ntbt_ms=1\n", env={})
    assert rows(daemon_part) == served(create_app(cfg, ControlPlane(cfg), background=False))
    assert rows(instance_part) == served(create_serving_app(None, ["m"]))
