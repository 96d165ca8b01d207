"""Configuration registry: sources, precedence, validation."""
import pytest

from crosspool_b200 import config as C

TOML = """
cache_root = "/tmp/cache"
[daemon]
port = 9999
[logging]
level = "warning"
[atn]
devices = [0, 1]
[ffn]
devices = [2, 3, 4]
[ffn.loader]
parallelism = 8
[scheduler]
ffn_concurrency = 2
ffn_policy = "random"
[scheduler.slo]
ttft_ms = 1000
tbt_ms = 50
[[models]]
id = "Qwen/Qwen3-8B"
path = "/models/q8"
atn_tp_size = 2
ffn_tp_size = 2
[[models]]
id = "Qwen/Qwen3-0.6B"
slo = { ttft_ms = 500, tbt_ms = 20 }
"""


def test_precedence_cli_over_env_over_toml_over_default():
    cfg = C.load_config(cli={"logging_level": "debug"}, env={"XPOOL_LOG_LEVEL": "error",
                        "XPOOL_FFN_LOADER_PARALLELISM": "16"}, toml_text=TOML)
    assert cfg.logging_level == "debug" and cfg.sources["logging_level"] == "cli"
    assert cfg.ffn_loader_parallelism == 16 and cfg.sources["ffn_loader_parallelism"] == "env"
    assert cfg.daemon_port == 9999 and cfg.sources["daemon_port"] == "toml"
    assert cfg.daemon_host == "127.0.0.1" and cfg.sources["daemon_host"] == "default"
    assert cfg.atn_devices == (0, 1) and cfg.ffn_devices == (2, 3, 4)
    assert cfg.scheduler_ffn_policy == "random" and cfg.scheduler_ffn_concurrency == 2


def test_models_and_slo_overrides():
    cfg = C.load_config(env={}, toml_text=TOML)
    assert [m.id for m in cfg.models] == ["Qwen/Qwen3-8B", "Qwen/Qwen3-0.6B"]
    assert cfg.ffn_tp_for("Qwen/Qwen3-8B") == 2
    assert cfg.ffn_tp_for("Qwen/Qwen3-0.6B") == 3  # default: all FFN devices
    assert cfg.slo_for("Qwen/Qwen3-8B") == C.Slo(1000, 50)
    assert cfg.slo_for("Qwen/Qwen3-0.6B") == C.Slo(500, 20)


def test_digest_is_stable_and_sensitive():
    a = C.load_config(env={}, toml_text=TOML)
    b = C.load_config(env={}, toml_text=TOML)
    c = C.load_config(env={}, toml_text=TOML.replace("9999", "9998"))
    assert a.digest() == b.digest() != c.digest()


@pytest.mark.parametrize("bad,msg", [
    (TOML.replace("devices = [2, 3, 4]", "devices = [1, 2]"), "both"),
    (TOML.replace("[scheduler.slo]\nttft_ms = 1000\ntbt_ms = 50", ""), "scheduler.slo"),
    (TOML.replace('ffn_policy = "random"', 'ffn_policy = "lifo"'), "ffn_policy"),
    (TOML.replace("atn_tp_size = 2", "atn_tp_size = 2\natn_dp_size = 2"), "TP-by-DP"),
    (TOML.replace('id = "Qwen/Qwen3-0.6B"', 'id = "Qwen/Qwen3-8B"'), "duplicate"),
    (TOML.replace("port = 9999", "port = 0"), "daemon.port"),
])
def test_rejections(bad, msg):
    with pytest.raises(C.ConfigError, match=msg):
        C.load_config(env={}, toml_text=bad)


def test_observer_env_switches():
    cfg = C.load_config(env={"XPOOL_DEBUG_FABRIC_OBSERVER_ENABLE": "1",
                             "XPOOL_DEBUG_FABRIC_OBSERVER_RECORD_CAPACITY": "128"}, toml_text=TOML)
    assert cfg.debug_fabric_observer_enable is True and cfg.debug_fabric_observer_record_capacity == 128
    assert cfg.debug_graph_observer_enable is False


def test_engine_knobs_and_ports_are_registry_settings_covered_by_the_digest():
    base = "[atn]\ndevices=[0]\n[ffn]\ndevices=[1]\n[scheduler.slo]\nttft_ms=1000\ntbt_ms=50\n"
    a = C.load_config(toml_text=base, env={})
    assert (a.engine_max_rows, a.engine_max_batch, a.engine_prefill_chunk, a.engine_page_size) == (4096, 256, 4096, 16)
    assert (a.serving_base_port, a.serving_tp_rendezvous_base_port) == (30000, 30500)
    b = C.load_config(toml_text=base + "[engine]\nmax_batch=64\npage_size=64\n[serving]\nbase_port=31000\n", env={"XPOOL_MAX_ROWS": "512"})
    assert (b.engine_max_rows, b.engine_max_batch, b.engine_page_size, b.serving_base_port) == (512, 64, 64, 31000)
    assert b.sources["engine_max_rows"] == "env" and b.sources["engine_max_batch"] == "toml"
    assert a.digest() != b.digest()      # two processes that disagree on slot sizing fail the config check
    with pytest.raises(C.ConfigError, match="page_size"):
        C.load_config(toml_text=base + "[engine]\npage_size=48\n", env={})


def test_model_paths_resolve_against_the_vendor_base_and_ids_must_be_canonical(tmp_path):
    import json

    import pytest

    from crosspool_b200 import config as C
    from crosspool_b200.runtime.backends import checkpoint_dir_for

    base = tmp_path / "models"
    (base / "acme" / "tiny").mkdir(parents=True)
    hf = {"architectures": ["Qwen3ForCausalLM"], "hidden_size": 64, "num_hidden_layers": 2, "num_attention_heads": 4,
          "num_key_value_heads": 2, "intermediate_size": 128, "vocab_size": 256, "head_dim": 16}
    (base / "acme" / "tiny" / "config.json").write_text(json.dumps(hf))
    (base / "acme" / "tiny" / "model.safetensors").write_bytes(b"")
    toml = f"""
[vendor]
model_base_uri = "{base}"
[atn]
devices = [0]
[ffn]
devices = [1]
[scheduler.slo]
ttft_ms = 2000
tbt_ms = 50
[[models]]
id = "acme/tiny"
[[models]]
id = "Qwen/Qwen3-0.6B"
[[models]]
id = "elsewhere"
path = "{tmp_path}/absolute"
"""
    cfg = C.load_config(toml_text=toml, env={})
    assert cfg.model_path("acme/tiny") == base / "acme" / "tiny"            # the id, under the base
    assert cfg.model_shape("acme/tiny").hidden_size == 64
    assert checkpoint_dir_for(cfg, "acme/tiny") == str(base / "acme" / "tiny")
    assert cfg.model_path("Qwen/Qwen3-0.6B") is None and cfg.model_shape("Qwen/Qwen3-0.6B").num_layers == 28   # a preset
    assert cfg.model_path("elsewhere") == tmp_path / "absolute"              # absolute paths ignore the base
    with pytest.raises(C.ConfigError, match="elsewhere"):
        cfg.model_shape("elsewhere")
    for bad in ("org/a/b", "../x", " org/model"):
        with pytest.raises(C.ConfigError, match="invalid model id"):
            C.load_config(toml_text=toml.replace('id = "acme/tiny"', f'id = "{bad}"'), env={})
