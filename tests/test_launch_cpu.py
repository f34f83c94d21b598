"""Host logic of the multi-rank launcher: per-rank environment, engine command line, early give-up when a
rank dies during start-up, teardown by the ranks' own PIDs (reference: tools/launch_occamy_ep.sh:51-131)."""
import subprocess
import sys
import time
from types import SimpleNamespace

from coffin_b200.tools import launch


def test_rank_env_and_engine_command_line():
    env = launch.rank_env(2, 4, 29511, "ep", base={"PATH": "/bin", "RANK": "9"})
    assert env["RANK"] == "2" and env["LOCAL_RANK"] == "2" and env["WORLD_SIZE"] == "4"
    assert env["MASTER_ADDR"] == "127.0.0.1" and env["MASTER_PORT"] == "29511" and env["COFFIN_PARALLEL"] == "ep"
    assert env["PATH"] == "/bin" and "CUDA_VISIBLE_DEVICES" not in env     # every rank sees every GPU (peer memory)
    argv = launch.engine_argv(SimpleNamespace(sock="/tmp/x.sock", model="/ckpt", preset=None), ["--max-seq", "4096"])
    assert argv[:4] == [sys.executable, "-m", "coffin_b200.entrypoints.cli.runtime", "--serve"]
    assert argv[4:] == ["--sock", "/tmp/x.sock", "--model", "/ckpt", "--max-seq", "4096"]
    assert 1024 < launch.free_port() < 65536


def test_start_up_gives_up_when_a_rank_has_exited(tmp_path, capsys):
    alive = subprocess.Popen([sys.executable, "-c", "import time; time.sleep(30)"])
    dead = subprocess.Popen([sys.executable, "-c", "import sys; sys.exit(7)"])
    dead.wait(10)
    t0 = time.monotonic()
    try:
        assert launch.wait_ping(str(tmp_path / "none.sock"), 20.0, [alive, dead]) is False
        assert time.monotonic() - t0 < 5.0 and "rank(s) [1] exited" in capsys.readouterr().err
        # nobody listens and nobody died: the limit itself ends the wait
        assert launch.wait_ping(str(tmp_path / "none.sock"), 1.0, [alive]) is False
    finally:
        launch.stop([alive, dead], grace=5.0)
    assert alive.poll() is not None


def test_stop_kills_a_rank_that_ignores_sigterm():
    stubborn = subprocess.Popen([sys.executable, "-c",
                                 "import signal, time; signal.signal(signal.SIGTERM, signal.SIG_IGN); print('up', flush=True); time.sleep(60)"],
                                stdout=subprocess.PIPE, text=True)
    assert stubborn.stdout.readline().strip() == "up"
    t0 = time.monotonic()
    launch.stop([stubborn], grace=1.0)
    stubborn.wait(5)
    assert stubborn.returncode is not None and time.monotonic() - t0 < 6.0


def test_runtime_cli_accepts_the_reference_flag_names():
    """Flags of the reference's command line that map onto this engine's options (or are accepted and ignored)."""
    import pytest
    from coffin_b200.entrypoints.cli.runtime import engine_config, parser
    args = parser().parse_args(["--serve", "--spec-min-ctx", "512", "--image-max-pixels", "500000", "--image-min-pixels", "4096",
                                "--max-images", "2", "--max-image-bytes", "1000", "--block-size", "64", "--fp16", "--no-bench",
                                "--backend", "auto", "--vision-int8"])
    cfg = engine_config(args)
    assert (cfg.spec_min_ctx, cfg.image_max_pixels, cfg.image_min_pixels, cfg.max_images, cfg.max_image_bytes) == \
        (512, 500000, 4096, 2, 1000)
    a = parser().parse_args(["generate", "--prompt", "hello", "--max-new", "7", "--print-ids"])
    assert a.cmd == "generate" and a.prompt == "hello" and a.n == 7 and a.print_ids
    a = parser().parse_args(["chat", "--user", "hi", "--think"])
    assert a.user == "hi" and a.think and not a.no_thinking
    for bad in (["--block-size", "32"], ["--backend", "corex"], ["--fp16", "--quant", "int8"]):
        with pytest.raises(SystemExit):
            engine_config(parser().parse_args(["--serve", *bad]))
