"""No-GPU checks of the boundary: the library loads, exports every declared symbol, the
ctypes structures match the header, and the host-side argument checks fail loudly."""
import ctypes as C
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    from nsa_from_scratch_b200 import _lib
    lib = _lib.load()
    header = open(os.path.join(ROOT, "include", "nsa_b200.h")).read()
    declared = set(re.findall(r"^(?:int|int64_t|const char\*)\s+(\w+)\s*\(", header, flags=re.M))
    assert declared, "no declarations parsed"
    assert declared == set(_lib.PROTOTYPES), declared ^ set(_lib.PROTOTYPES)
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.nsa_abi_version() == 7


def _struct_fields(header, name):
    body = re.search(r"typedef struct %s \{(.*?)\} %s;" % (name, name), header, flags=re.S).group(1)
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    out = []
    for decl in body.split(";"):
        decl = decl.strip()
        if not decl:
            continue
        names = [n.strip().lstrip("*") for n in decl.split(",")]
        names[0] = names[0].split()[-1].lstrip("*")
        out += names
    return out


def test_ctypes_structs_match_header():
    from nsa_from_scratch_b200 import _lib
    header = open(os.path.join(ROOT, "include", "nsa_b200.h")).read()
    assert [f[0] for f in _lib.FwdArgs._fields_] == _struct_fields(header, "nsa_fwd_args")
    assert [f[0] for f in _lib.BwdArgs._fields_] == _struct_fields(header, "nsa_bwd_args")


def test_argument_errors_are_reported_without_a_gpu():
    from nsa_from_scratch_b200 import _lib
    lib = _lib.load()
    a = _lib.FwdArgs()
    assert lib.nsa_attention_fwd(C.byref(a), None) == -1            # NULL Q
    assert b"NULL" in lib.nsa_last_error()
    assert lib.nsa_pool_mean(1, 1, 1, 1, 64, 60, 32, 32, 2, 0, 1.0, None) == -1   # D not a multiple of 8
    assert b"multiple of 8" in lib.nsa_last_error()
    assert lib.nsa_attention_fwd(None, None) == -1
    ERR_ARG, ERR_UNSUPPORTED = -1, -2
    # every entry point added around the path checks its arguments before it touches the device
    assert lib.nsa_rope_to_heads(None, 1, None, None, 1, 8, 2, 64, 2, 2, 0, None) == ERR_ARG
    assert lib.nsa_rope_to_heads(1, 1, 1, None, 1, 8, 2, 64, 2, 2, 0, None) == ERR_ARG           # cos without sin
    assert lib.nsa_rope_to_heads(1, 1, None, None, 1, 8, 2, 24, 2, 2, 0, None) == ERR_UNSUPPORTED  # D % 16
    assert b"multiple of 16" in lib.nsa_last_error()
    assert lib.nsa_memcpy_2d(1, 8, 1, 16, 16, 2, 1, None) == ERR_ARG                              # pitch < row
    assert lib.nsa_memcpy_2d(1, 16, 1, 16, 16, 2, 7, None) == ERR_ARG
    assert lib.nsa_cache_append(1, 1, 1, 1, 1, 1, 1, 1, 1, 64, 4, 62, 64, 8, 1, 32, 16, 64, 0, None) == ERR_ARG   # 62 + 4 > 64
    assert b"exceed the allocation" in lib.nsa_last_error()
    assert lib.nsa_cache_append_dev(1, 1, 1, 1, 1, 1, 1, 1, 1, 64, 1, None, 64, 8, 1, 32, 16, 64, 0, None) == ERR_ARG
    assert lib.nsa_select_blocks_cached(1, 1, 1, 1, 4, 1, 1, 8, 64, 4, 64, 64, None, 0.125, 0, 0, 0, 0, None) == ERR_ARG
    assert lib.nsa_cmp_block_scores_tc(1, 1, 1, 1, 1, 1, 4, 1, 256, 15, 32, 4, 32, 16, 0, 64, 0, 1, 0.2, 0, 0, 0, 0, None) == ERR_UNSUPPORTED
    assert b"tcgen05" in lib.nsa_last_error()                                                      # D = 32
    assert lib.nsa_cmp_block_scores(1, 1, None, 1, 1, 4, 1, 256, 15, 64, 4, 32, 16, 0, 64, 0, 1, 0.125, 0, 0, 0, 0, None) == ERR_ARG
    b = _lib.FwdArgs()
    b.Q = b.out = b.K = b.V = 1
    b.B, b.H, b.Hkv, b.Tq, b.Tk, b.D = 1, 4, 1, 64, 64, 64
    b.branches, b.fused, b.window, b.q_dtype, b.kv_dtype = 4, 1, 16, 0, 0
    b.nsplit = 17
    assert lib.nsa_attention_fwd(C.byref(b), None) == ERR_ARG and b"nsplit" in lib.nsa_last_error()
    b.nsplit, b.io_layout = 0, 8
    assert lib.nsa_attention_fwd(C.byref(b), None) == ERR_ARG and b"io_layout" in lib.nsa_last_error()
    b.io_layout, b.fused, b.accumulate = 0, 0, 1
    assert lib.nsa_attention_fwd(C.byref(b), None) == ERR_ARG and b"accumulate" in lib.nsa_last_error()
    # K/V share Q's type, or are bf16 beside an fp8 Q -- nothing else
    b.accumulate, b.q_dtype, b.kv_dtype = 0, 0, 2
    assert lib.nsa_attention_fwd(C.byref(b), None) == ERR_UNSUPPORTED and b"K/V dtype" in lib.nsa_last_error()
    b.q_dtype, b.kv_dtype = 2, 1
    assert lib.nsa_attention_fwd(C.byref(b), None) == ERR_UNSUPPORTED and b"K/V dtype" in lib.nsa_last_error()
    assert lib.nsa_fp8_dequantize(None, 16, 16, 2, 1.0, None) == ERR_ARG
    assert lib.nsa_fp8_dequantize(16, 16, 16, 0, 1.0, None) == ERR_ARG and b"format" in lib.nsa_last_error()
    assert lib.nsa_fp8_dequantize(16, 16, 16, 2, 0.0, None) == ERR_ARG and b"scale" in lib.nsa_last_error()
    assert lib.nsa_fp8_dequantize(16, 24, 16, 2, 1.0, None) == ERR_ARG and b"aligned" in lib.nsa_last_error()
    assert lib.nsa_fp8_dequantize(16, 16, -1, 2, 1.0, None) == ERR_ARG


def test_no_cpu_fallback():
    import nsa_from_scratch_b200 as nsa
    x = torch.zeros(1, 1, 64, 64, dtype=torch.bfloat16)
    with pytest.raises((RuntimeError, AssertionError)):
        nsa.sliding_attention(x, x, x)
    with pytest.raises((RuntimeError, AssertionError)):
        nsa.nsa_forward(x, x, x, nsa.NSAConfig())


def test_compat_shim_maps_reference_module_names():
    from nsa_from_scratch_b200 import compat
    compat.install()
    import nsa.cuda as nc
    import nsa.triton.forward as nf
    import nsa.triton.selected as ns
    assert nf.nsa_forward.__module__.startswith("nsa_from_scratch_b200")
    assert ns.selected_attention.__module__.startswith("nsa_from_scratch_b200")
    ext = nc._get_ext()
    assert hasattr(ext, "selected_attention_fwd_cuda") and hasattr(ext, "selected_attention_bwd_cuda")


def test_host_pipeline_chunking_rules():
    """Query chunks of the host-tensor entry point exist only where every block grid lines up at the chunk
    boundaries; anything else is one chunk."""
    from nsa_from_scratch_b200.config import NSAConfig
    from nsa_from_scratch_b200.host import _chunk_rows
    cfg = NSAConfig(block_size_c=32, stride_c=16, top_k=16, window_size=512)
    assert _chunk_rows(cfg, 65536, 65536, 16384) == 16384
    assert _chunk_rows(cfg, 65536, 65536, 10000) == 9984          # rounded down to a multiple of 64
    assert _chunk_rows(cfg, 65536, 65536, None) == 65536
    assert _chunk_rows(cfg, 65500, 65500, 16384) == 65500         # ragged tail: one chunk
    assert _chunk_rows(cfg, 4096, 2048, 1024) == 4096             # more queries than keys: one chunk
    assert _chunk_rows(NSAConfig(causal=False), 4096, 4096, 1024) == 4096
    assert _chunk_rows(NSAConfig(block_size_c=96), 768 * 4, 768 * 4, 1000) == 960       # multiples of lcm(64, 96) = 192


def test_compat_fused_caller_keeps_the_cpu_route():
    """compat.install(fuse_caller=True) patches the reference's attention module when it is importable; CPU
    inputs (and anything under autograd) still run the module's own code, bit for bit."""
    import os
    import sys
    ref = os.environ.get("NSA_REFERENCE_CHECKOUT", "")
    if not ref:                                   # default: a checkout named "reference" beside this repository
        ref = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")
    if not os.path.isdir(os.path.join(ref, "nsa", "model")):
        pytest.skip("reference checkout not present")
    sys.path.insert(0, ref)
    saved = {k: sys.modules.pop(k) for k in list(sys.modules) if k == "nsa" or k.startswith("nsa.")}   # an earlier shim, if any
    try:
        import torch
        from nsa.model.config import TransformerConfig
        from nsa.model.llama_dense import _build_rope_cache
        from nsa.model.llama_nsa import NSAAttention
        torch.manual_seed(0)
        cfg = TransformerConfig(n_heads=2, head_dim=32, hidden_size=48, nsa_block_size_c=32, nsa_top_k=2, nsa_window_size=32)
        mod = NSAAttention(cfg)
        x = torch.randn(1, 128, 48)
        cos, sin = _build_rope_cache(128, 32, cfg.rope_theta, "cpu", torch.float32)
        with torch.no_grad():
            before = mod(x, cos, sin)
        from nsa_from_scratch_b200 import compat
        compat.install(fuse_caller=True)
        assert getattr(NSAAttention.forward, "_b200_token_major", False)
        with torch.no_grad():
            after = mod(x, cos, sin)
        assert torch.equal(torch.nan_to_num(before), torch.nan_to_num(after))
    finally:
        sys.path.remove(ref)
        for k in [k for k in sys.modules if k == "nsa" or k.startswith("nsa.")]:
            del sys.modules[k]
        sys.modules.update(saved)
