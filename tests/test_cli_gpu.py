"""Runs the C++ operator test programs (tests/cli), the counterparts of the
reference's op_test_flash_attn and op_test_rope_single command-line tests, with
the reference's flags.  They exercise the C++ host layer (Tensor, GPUAllocator)
and the C ABI from C++ and compare with the CPU checker."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
CLI = os.path.join(HERE, "cli")


@pytest.fixture(scope="module")
def binaries():
    env = dict(os.environ)
    env.pop("CXX", None)
    subprocess.check_call(["make", "-C", CLI], env=env, stdout=subprocess.DEVNULL)
    return os.path.join(CLI, "bin")


def run(binary, *args):
    r = subprocess.run([binary] + [str(a) for a in args], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "test success" in r.stdout
    return r.stdout


@pytest.mark.parametrize("args", [
    ("--m", 256, "--n", 256, "--offset", 0, "--head_num", 32, "--head_dim", 128),   # Llama-2-7B-shaped prefill
    ("--m", 1, "--n", 700, "--offset", 699, "--head_num", 32),                       # decode shape
    ("--m", 300, "--n", 812, "--offset", 512, "--head_num", 4, "--mode", "strict"),
    ("--m", 200, "--n", 200, "--group_size", 5, "--kv_head_num", 2, "--dtype", "bfloat16"),
    (),                                                                             # the reference's defaults: m = n = 2048, 32 heads
    ("--m", 4096, "--n", 8192, "--offset", 4096, "--head_num", 4),                  # a 4096-token chunk behind 4096 cached tokens
    ("--m", 4096, "--n", 8192, "--offset", 4096, "--group_size", 5, "--kv_head_num", 1, "--dtype", "bfloat16"),
])
def test_flash_attn_main(binaries, args):
    out = run(os.path.join(binaries, "flash_attn_main"), *args)
    assert "beyond: 0)" in out
    if "bfloat16" not in args:        # fp16: no element needs the one-ulp term, and the reference's own verdict holds
        assert out.count("within(1e-2,1e-3) yes") == 2 and "above 1e-2: 0 of" in out
        assert "reference all_close(1e-3, 1e-3) on the fp32 golden: yes" in out


@pytest.mark.parametrize("args", [
    ("--dtype", "float16"),                                                           # reference defaults
    ("--dtype", "bfloat16", "--seq_len", 77, "--offset", 4000, "--head_num", 12),
    ("--dtype", "float16", "--is_neox", "false", "--seq_len", 1, "--offset", 5, "--head_num", 40),
])
def test_rope_single_layer_main(binaries, args):
    out = run(os.path.join(binaries, "rope_single_layer_main"), *args)
    assert "bit-identical: yes" in out


@pytest.mark.parametrize("args", [
    ("--arch", "qwen2"),                                                   # 12 query heads on 2 KV heads, bf16, neox pairs
    ("--arch", "qwen2", "--kv_head_num", 8, "--group_size", 5, "--prompt", 700, "--steps", 3),
    ("--arch", "llama2"),                                                  # 8 heads MHA, fp16, interleaved pairs
    ("--arch", "llama2", "--kv_head_num", 32, "--prompt", 256, "--dtype", "bfloat16"),
])
def test_attention_section_with_reference_names(binaries, args):
    """The reference's call sequence under its own operator names (include/npu_ops_compat.hpp)."""
    out = run(os.path.join(binaries, "npu_names_main"), *args)
    assert "caches bit-identical to the checker: yes" in out and "error handler calls: 1" in out
