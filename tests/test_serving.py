"""Serving adapters for an exported drafter: configuration, export contract, server life-cycle and the response gate,
against a stand-in HTTP server (no SGLang / vLLM needed)."""
import json
import sys
import threading
from http.server import BaseHTTPRequestHandler, HTTPServer

import pytest

from turbo_dllm_b200.serving import dflash_servers as srv


def _good_response(model="draft-served", n=15, text="a b c d e f g h i j k l m n o p"):
    hist = [0] * (n + 1)
    hist[n] = 2
    return {"model": model, "choices": [{"text": text}],
            "metrics": {"speculative_decoding": {"num_spec_tokens": n, "num_spec_steps": 3,
                                                 "num_accepted_draft_tokens": 2 * n, "num_draft_tokens": 3 * n,
                                                 "acceptance_histogram": hist}}}


def test_server_config_normalises_aliases_and_builds_both_commands():
    v = srv.ServerConfig.from_mapping({"backend": "vllm", "model": "T", "draft": "D", "tp": 2, "block_size": 8,
                                       "gpu_memory_utilization": 0.8, "max_model_len": 4096})
    cmd = v.command()
    assert cmd[:3] == ["vllm", "serve", "T"] and v.port == 8000 and v.url == "http://127.0.0.1:8000"
    spec = json.loads(cmd[cmd.index("--speculative-config") + 1])
    assert spec == {"method": "dflash", "model": "D", "num_speculative_tokens": 7}
    assert cmd[cmd.index("--gpu-memory-utilization") + 1] == "0.8" and "--max-model-len" in cmd
    s = srv.ServerConfig.from_mapping({"backend": "sglang", "target_model": "T", "draft_export": "D",
                                       "mem_fraction_static": 0.7})
    c = s.command()
    assert s.port == 30000 and c[c.index("--speculative-num-draft-tokens") + 1] == "15"
    assert c[c.index("--mem-fraction-static") + 1] == "0.7"
    with pytest.raises(ValueError, match="unknown server setting"):
        srv.ServerConfig.from_mapping({"backend": "vllm", "model": "T", "draft": "D", "speed": 11})
    with pytest.raises(ValueError, match="block_size"):
        srv.ServerConfig.from_mapping({"backend": "vllm", "model": "T", "draft": "D", "block_size": 1})


def test_version_requirement_and_export_contract(tmp_path):
    assert srv.require_server_version("vllm", "0.29.0") == "0.29.0"
    with pytest.raises(RuntimeError, match="qualified release"):
        srv.require_server_version("vllm", "0.22.0")
    assert srv.require_server_version("sglang", "0.5") == "0.5"
    d = tmp_path / "export"
    d.mkdir()
    with pytest.raises(ValueError, match="no config.json"):
        srv.validate_export_for_server(str(d), "vllm")
    cfg = {"model_type": "qwen3", "architectures": ["DFlash2DraftModel"], "block_size": 16,
           "dflash_config": {"block_size": 16}}
    (d / "config.json").write_text(json.dumps(cfg))
    with pytest.raises(ValueError, match="no weight file"):
        srv.validate_export_for_server(str(d), "vllm")
    (d / "model.safetensors").write_bytes(b"x")
    assert srv.validate_export_for_server(str(d), "vllm", 16)["num_speculative_tokens"] == 15
    with pytest.raises(ValueError, match="expected 8"):
        srv.validate_export_for_server(str(d), "vllm", 8)
    (d / "config.json").write_text(json.dumps({**cfg, "dflash_config": {"block_size": 8}}))
    with pytest.raises(ValueError, match="conflicting block sizes"):
        srv.validate_export_for_server(str(d), "sglang")
    (d / "config.json").write_text(json.dumps({**cfg, "model_type": "llama"}))
    with pytest.raises(ValueError, match="model_type 'qwen3' only"):
        srv.validate_export_for_server(str(d), "vllm")
    assert srv.validate_export_for_server(str(d), "sglang")["block_size"] == 16


def test_response_gate_names_every_shortfall():
    models = {"data": [{"id": "draft-served"}]}
    expected = "a b c d e f g h i j k l m n o p q"
    ok = srv.evaluate_response(models=models, response=_good_response(), model="draft-served", expected_text=expected,
                               encode=str.split, block_size=16)
    assert ok["passed"] and ok["target_prefix_match_tokens"] == 16 and ok["full_blocks_accepted"] == 2
    bad = _good_response(text="a b c x")
    bad["metrics"]["speculative_decoding"].update(num_spec_tokens=7, acceptance_histogram=[1] * 8)
    res = srv.evaluate_response(models={"data": []}, response=bad, model="draft-served", expected_text=expected,
                                encode=str.split, block_size=16)
    joined = " | ".join(res["errors"])
    assert not res["passed"]
    for part in ("is not served", "drafts 7 tokens", "no complete draft block", "target prefix match 3 < draft length 15"):
        assert part in joined
    # SGLang puts its counters beside the completion
    sg = {"model": "draft-served", "choices": [{"text": expected, "meta_info": {
        "spec_num_draft_tokens": 15, "spec_verify_ct": 2, "spec_accepted_tokens": 20, "spec_draft_tokens": 30,
        "spec_accept_histogram": [0] * 15 + [1]}}]}
    assert srv.evaluate_response(models=models, response=sg, model="draft-served", expected_text=expected,
                                 encode=str.split, block_size=16)["passed"]
    none = srv.evaluate_response(models=models, response={"model": "draft-served", "choices": [{"text": expected}]},
                                 model="draft-served", expected_text=expected, encode=str.split, block_size=16)
    assert "no speculative-decoding counters" in " ".join(none["errors"])


class _Handler(BaseHTTPRequestHandler):
    def _send(self, obj):
        body = json.dumps(obj).encode()
        self.send_response(200)
        self.send_header("Content-Type", "application/json")
        self.send_header("Content-Length", str(len(body)))
        self.end_headers()
        self.wfile.write(body)

    def do_GET(self):   # noqa: N802
        self._send({"data": [{"id": "draft-served"}]})

    def do_POST(self):   # noqa: N802
        req = json.loads(self.rfile.read(int(self.headers["Content-Length"])))
        assert req["temperature"] == 0.0 and req["max_tokens"] >= 15 and not req["stream"]
        self._send(_good_response(model=req["model"]))

    def log_message(self, *a):
        pass


def test_verify_against_a_running_endpoint():
    httpd = HTTPServer(("127.0.0.1", 0), _Handler)
    t = threading.Thread(target=httpd.serve_forever, daemon=True)
    t.start()
    try:
        url = f"http://127.0.0.1:{httpd.server_address[1]}"
        res = srv.verify_server(server_url=url, model="draft-served", prompt="say the alphabet",
                                expected_text="a b c d e f g h i j k l m n o p q", encode=str.split, block_size=16)
        assert res["passed"], res
        with pytest.raises(ValueError, match="cover one draft block"):
            srv.verify_server(server_url=url, model="m", prompt="p", expected_text="e", encode=str.split, block_size=16,
                              max_tokens=3)
    finally:
        httpd.shutdown()


SERVER = """
import json, sys
from http.server import BaseHTTPRequestHandler, HTTPServer
class H(BaseHTTPRequestHandler):
    def do_GET(self):
        b = json.dumps({"data": [{"id": "stand-in"}]}).encode()
        self.send_response(200); self.send_header("Content-Length", str(len(b))); self.end_headers(); self.wfile.write(b)
    def log_message(self, *a): pass
HTTPServer(("127.0.0.1", int(sys.argv[1])), H).serve_forever()
"""


def test_server_process_starts_waits_and_stops_its_own_process(tmp_path):
    import socket

    with socket.socket() as so:
        so.bind(("127.0.0.1", 0))
        port = so.getsockname()[1]
    script = tmp_path / "server.py"
    script.write_text(SERVER)
    sp = srv.ServerProcess([sys.executable, str(script), str(port)], f"http://127.0.0.1:{port}",
                           log_path=str(tmp_path / "server.log"))
    with sp as running:
        models = running.wait_ready(timeout=30, poll=0.1)
        assert models["data"][0]["id"] == "stand-in"
        pid = running.proc.pid
        assert pid > 0
    assert sp.proc is None
    # a command that exits before answering is reported, not waited for
    dead = srv.ServerProcess([sys.executable, "-c", "raise SystemExit(3)"], f"http://127.0.0.1:{port}").start()
    with pytest.raises(RuntimeError, match="exited with code 3"):
        dead.wait_ready(timeout=10, poll=0.1)
    dead.stop()


def test_cli_prints_the_command_and_verifies(capsys):
    from turbo_dllm_b200.cli.dflash import run_dflash

    assert run_dflash(["serve-vllm", "--target-model", "T", "--draft", "D", "--block-size", "8", "--tp", "2"]) == 0
    out = capsys.readouterr().out
    assert "vllm serve T" in out and '"num_speculative_tokens": 7' in out
    httpd = HTTPServer(("127.0.0.1", 0), _Handler)
    threading.Thread(target=httpd.serve_forever, daemon=True).start()
    try:
        url = f"http://127.0.0.1:{httpd.server_address[1]}"
        rc = run_dflash(["verify-vllm", "--base-url", url, "--model", "draft-served", "--prompt", "p",
                         "--expected-text", "a b c d e f g h i j k l m n o p q"])
        assert rc == 0 and json.loads(capsys.readouterr().out)["passed"]
    finally:
        httpd.shutdown()
