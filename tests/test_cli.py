import json

from crosspool_b200 import config as C
from crosspool_b200.cli import main as cli


def test_config_dump_and_memory_profile(tmp_path, capsys, monkeypatch):
    monkeypatch.delenv("XPOOL_CONFIG", raising=False)
    assert cli.main(["--config", "configs/xpool.example.toml", "--log-level", "debug", "config", "dump"]) == 0
    out = json.loads(capsys.readouterr().out)
    assert out["config"]["logging_level"] == "debug" and out["sources"]["logging_level"] == "cli"
    assert out["config"]["ffn_devices"] == [2, 3, 4, 5, 6, 7] and len(out["config"]["models"]) == 3
    assert cli.main(["--config", "configs/xpool.example.toml", "memory-profile"]) == 0
    prof = json.loads(capsys.readouterr().out)
    assert set(prof["devices"]) == {"2", "3", "4", "5", "6", "7"}
    big = [g for g in prof["groups"] if g["model_id"] == "Qwen/Qwen3-32B"]
    assert big and len(big[0]["devices"]) == 4
    assert all(d["headroom"] >= 0 for d in prof["devices"].values())


def test_exec_environment_exports_devices_and_endpoint():
    cfg = C.load_config(cli={"config": "configs/xpool.example.toml"}, env={})
    env = cli.exec_environment(cfg, {"PATH": "/bin"})
    assert env["CUDA_VISIBLE_DEVICES"] == "0,1,2,3,4,5,6,7"
    assert env["XPOOL_DAEMON_PORT"] == "9810" and env["XPOOL_CONFIG"].endswith("xpool.example.toml")
    assert env["SGLANG_PLUGINS"] == "xpool" and env["PATH"] == "/bin"


def test_missing_required_settings_exit_2(capsys, monkeypatch):
    monkeypatch.delenv("XPOOL_CONFIG", raising=False)
    assert cli.main(["memory-profile"]) == 2
    assert "configuration error" in capsys.readouterr().err


def test_qualify_subcommand_passes_option_like_arguments_through(capsys):
    from crosspool_b200.cli import main as cli

    assert cli.main(["qualify", "--arch", "Qwen2ForCausalLM"]) == 0
    assert "Qwen2ForCausalLM: PASS" in capsys.readouterr().out
