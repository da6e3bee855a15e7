"""CPU checks of the drop-in boundary: the library loads and exports every
symbol the public header declares; nothing is computed (no GPU here)."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols(header="gpu_ops.h"):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(gpu_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from llm_simple_b200 import ops
    lib = ctypes.CDLL(ops.LIB_PATH)
    names = declared_symbols()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), n
    assert sorted(ops.EXPORTS) == names


def test_library_exports_every_symbol_of_the_host_layer_header():
    from llm_simple_b200 import layer, ops
    lib = ctypes.CDLL(ops.LIB_PATH)
    names = declared_symbols("gpu_layer.h")
    for n in names:
        assert hasattr(lib, n), n
    assert sorted(layer.EXPORTS) == names


def test_descriptor_struct_matches_the_header_layout():
    from llm_simple_b200 import ops
    # 6 x int32 then 10 x int64, no padding
    assert ctypes.sizeof(ops.AttnDesc) == 6 * 4 + 10 * 8
    assert ops.AttnDesc.q_seq_stride.offset == 24
    d = ops.make_desc(ops.DT_BFLOAT16, 2, 40, 8, 1, 4096, layout="head")
    assert (d.cache_head_stride, d.cache_pos_stride, d.cache_seq_stride) == (4096 * 128, 128, 8 * 4096 * 128)
    t = ops.make_desc(ops.DT_FLOAT16, 1, 32, 32, 256, 256, layout="token")
    assert (t.cache_head_stride, t.cache_pos_stride) == (128, 32 * 128)


def test_data_type_values_are_the_reference_ones():
    text = open(os.path.join(ROOT, "include", "defs.hpp")).read()
    body = re.search(r"enum DataType[^{]*\{(.*?)\}", text, flags=re.S).group(1)
    names = [x.strip().split("=")[0].strip() for x in body.split(",") if x.strip()]
    assert names.index("DT_FLOAT16") == 4 and names.index("DT_BFLOAT16") == 5 and names.index("DT_FLOAT32") == 6


def test_host_side_validation_needs_no_gpu():
    from llm_simple_b200 import ops
    L = ops.lib()
    assert L.gpu_attn_set_decode_chunk(100) != 0
    assert b"multiple of 64" in L.gpu_ops_last_error_string()
    assert L.gpu_attn_set_decode_chunk(0) == 0
    assert L.gpu_flash_attn_layer(None, None, None, None, 4, 4, 0, 2, 64, 4, None) == -2
    assert L.gpu_attn_decode_workspace_bytes(None, 10) == 0


def test_reference_named_overloads_compile_and_link():
    """include/npu_ops_compat.hpp: the reference's operator names (prebuild/npu_ops.h:6-18, :27-30, :39-47) with
    its argument order, DataType and the stream by reference.  The test program written with those names compiles
    and links against the library here, without a GPU (it runs in the GPU suite)."""
    import subprocess
    cli = os.path.join(ROOT, "tests", "cli")
    env = dict(os.environ)
    env.pop("CXX", None)
    subprocess.check_call(["make", "-C", cli, "bin/npu_names_main"], env=env, stdout=subprocess.DEVNULL)
    assert os.path.exists(os.path.join(cli, "bin", "npu_names_main"))
    text = open(os.path.join(ROOT, "include", "npu_ops_compat.hpp")).read()
    for name in ("npu_flash_attn_layer", "npu_flash_attn_gqa_layer", "npu_flash_attn_opt_prefill_layer",
                 "npu_split_qkv_layer", "npu_rope_layer", "npu_rope_single_layer"):
        assert re.search(r"inline void %s\(" % name, text), name
    assert text.count("aclrtStream &stream") == 6
