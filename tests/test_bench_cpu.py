"""CPU checks of bench.py's bookkeeping: the algorithmic byte counts the roofline and the
throughput figures divide by (every operand once: Q4_K super-blocks of 144 bytes, Q8_1 blocks
of 36 bytes, F32 outputs), and the command line."""
import importlib.util
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_algorithmic_bytes_of_the_gemma_ffn_products():
    b = _bench()
    for batch in (1, 2, 4, 8):
        # fused gate/up: two 10240 x 2560 matrices, one Q8_1 row of 2560, 10240 F32 outputs
        assert b.glu_launch_bytes(batch) == 2 * 14_745_600 + 43_840 * batch
        # down: 2560 x 10240, one Q8_1 row of 10240, 2560 F32 outputs
        step = b.step_bytes(batch, layers=1)
        assert step - b.glu_launch_bytes(batch) == 14_745_600 + 21_760 * batch
        assert b.step_bytes(batch, layers=34) == 34 * step
    assert b.glu_launch_bytes(1, shard=2) == 14_745_600 + 2_880 + 5_120 * 4


def test_command_line_takes_the_contract_flags():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--help"],
                         capture_output=True, text=True, check=True).stdout
    for flag in ("--gpus", "--steps", "--warmup", "--impl", "--batch", "--workload", "--shard"):
        assert flag in out
