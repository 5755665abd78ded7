"""Host-side pieces of bench.py that need no GPU: the decoder leg's handling of its child processes and
the algorithmic byte count of the workload."""
import json
import subprocess
import types

import bench


def test_decoder_leg_parses_the_child_line(monkeypatch):
    def fake_run(cmd, **kw):
        batch = int(cmd[cmd.index("--batch") + 1])
        line = json.dumps({"metric": "27B EXL3 decode tokens/s", "value": 100.0 * batch, "ms_per_step": 10.0,
                           "status_word": 0})
        return types.SimpleNamespace(returncode=0, stdout="NCCL version x\n" + line + "\n", stderr="")
    monkeypatch.setattr(subprocess, "run", fake_run)
    out = bench.decoder_tok_s()
    assert out["unit"] == "tok/s" and out["bs1"]["value"] == 100.0 and out["bs32"]["value"] == 3200.0
    assert out["bs1"]["status_word"] == 0


def test_decoder_leg_never_raises(monkeypatch):
    monkeypatch.setattr(subprocess, "run", lambda cmd, **kw: types.SimpleNamespace(returncode=1, stdout="", stderr="boom"))
    out = bench.decoder_tok_s()
    assert "unavailable" in out["bs1"] and "unavailable" in out["bs32"]

    def hang(cmd, **kw):
        raise subprocess.TimeoutExpired(cmd, kw.get("timeout", 0))
    monkeypatch.setattr(subprocess, "run", hang)
    out = bench.decoder_tok_s()
    assert out["bs1"]["unavailable"].startswith("TimeoutExpired")
    monkeypatch.setattr(subprocess, "run", lambda cmd, **kw: types.SimpleNamespace(returncode=0, stdout="{not json", stderr=""))
    assert "unavailable" in bench.decoder_tok_s()["bs32"]


def test_algorithmic_bytes_of_the_workload():
    # trellis + activations in + activations out, per shard (5120 -> 6144 at 4 bpw, one row)
    assert bench.algorithmic_bytes(5120, [(6144, 4)], 1) == 5120 * 6144 * 4 // 8 + 5120 * 2 + 6144 * 2
    fused = bench.algorithmic_bytes(5120, [(17408, 3), (17408, 3)], 4)
    assert fused == 2 * (5120 * 17408 * 3 // 8) + 4 * 5120 * 2 + 4 * 2 * 17408 * 2
