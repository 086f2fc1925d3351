"""The C-ABI library loads, exports every symbol the header declares, and rejects bad
arguments on the host before anything is launched (no CUDA device needed)."""
import ctypes
import subprocess
import sys

import pytest


def test_every_declared_symbol_is_exported(pkg):
    L = pkg.lib()
    protos = pkg.parse_header()
    assert len(protos) >= 40
    dll = ctypes.CDLL(str(pkg._lib.LIB_PATH))
    for name in protos:
        assert hasattr(dll, name), name


def test_reference_names_are_present(pkg):
    # crates/triton-kernels/src/lib.rs:45-76 (the hot-path subset) + the two int4 GEMM examples
    names = set(pkg.parse_header())
    for n in ["rms_norm_f16", "rms_norm_f32", "fused_add_rms_norm_f16", "fused_add_rms_norm_f32",
              "residual_add_f16", "residual_add_f32", "residual_add_inplace_f16", "residual_add_inplace_f32",
              "fused_silu_mul_f16", "fused_silu_mul_f32", "fused_silu_mul_interleaved_f16",
              "fused_silu_mul_interleaved_f32", "rope_q_f32", "rope_k_f32", "rope_full_f32", "kv_cache_append_f32",
              "batched_decode_attention_f32", "batched_flash_decode_attn_phase1_f32", "flash_decode_attn_phase1_f32",
              "flash_decode_attn_phase2_f32", "w4a16_gptq_gemm_f16", "awq_gemm_int4_f16", "dequant_int4_to_fp16",
              "dequant_int4_sym_to_fp16", "decode_attention_f16", "decode_attention_hm_f16",
              "paged_decode_attention_f16"]:
        assert n in names, n


def test_argument_order_matches_reference(pkg):
    protos = pkg.parse_header()
    # w4a16_gptq_gemm_typed.rs:110-128 and awq_gemm_int4_typed.rs:96-114
    want = ["a", "qweight", "scales", "qzeros", "c", "m_size", "n_size", "k_size", "group_size", "stride_am",
            "stride_ak", "stride_qwk", "stride_qwn", "stride_sk", "stride_sn", "stride_qzk", "stride_qzn",
            "stride_cm", "stride_cn", "stream"]
    assert [n for _, n in protos["w4a16_gptq_gemm_f16"][1]] == want
    assert [n for _, n in protos["awq_gemm_int4_f16"][1]] == want
    # attention.rs:187-197
    assert [n for _, n in protos["decode_attention_hm_f16"][1]] == [
        "q", "k_cache", "v_cache", "output", "num_q_heads", "num_kv_heads", "head_dim", "capacity", "valid_kv_len",
        "scale", "stream"]
    # norms.rs:189-198
    assert [n for _, n in protos["fused_add_rms_norm_f16"][1]][:8] == [
        "input", "residual", "weight", "output", "residual_out", "hidden_size", "inv_n", "eps"]
    # cache.rs:22-30
    assert [n for _, n in protos["kv_cache_append_f32"][1]][:7] == [
        "new_keys", "new_values", "k_cache", "v_cache", "cache_idx", "num_heads", "head_dim"]


def test_host_side_rejections(pkg):
    L = pkg.lib()
    with pytest.raises(pkg.B200KError) as e:
        L.call("rms_norm_f16", None, None, None, 128, 1 / 128, 1e-5, 4, None)
    assert e.value.code == -1 and "NULL" in e.value.message
    with pytest.raises(pkg.B200KError) as e:
        L.call("w4a16_gptq_gemm_f16", 16, 16, 16, 16, 16, 4, 64, 100, 128, 100, 1, 64, 1, 64, 1, 8, 1, 64, 1, None)
    assert e.value.code == -2 and "group_size" in e.value.message
    with pytest.raises(pkg.B200KError) as e:
        L.call("decode_attention_f16", 16, 16, 16, 16, 32, 5, 128, 100, 0.1, None)
    assert e.value.code == -2
    with pytest.raises(pkg.B200KError) as e:
        L.call("fused_silu_mul_interleaved_f16", 16, 16, 96, 100, None)
    assert e.value.code == -2
    assert L.call("b200k_gemm_workspace_bytes", 16, 4096, 4096) > 0
    assert L.call("b200k_attention_workspace_bytes", 0, 32, 8, 128, 8192) == 0


def test_cpu_tensor_is_refused(P):
    import torch
    with pytest.raises((ValueError, RuntimeError, AssertionError)):
        P.residual_add_f32(torch.zeros(8), torch.zeros(8), torch.zeros(8), 8)


def test_missing_library_fails_loudly(pkg, tmp_path):
    with pytest.raises(FileNotFoundError):
        pkg.Library(tmp_path / "libb200_kernels.so")


def test_oracle_is_not_reachable_from_the_package():
    # the shipped package must not import or load the oracle
    code = ("import importlib,sys; sys.path.insert(0,'.'); importlib.import_module('triton-rs_b200'); "
            "assert not any(m == 'oracle' or m.startswith('oracle.') for m in sys.modules)")
    from conftest import ROOT
    subprocess.run([sys.executable, "-c", code], cwd=ROOT, check=True)
    for f in (ROOT / "triton-rs_b200").rglob("*"):
        if f.suffix in (".py", ".cu", ".cuh", ".h", ".cpp"):
            assert "oracle" not in f.read_text(), f


def test_rust_sys_binding_is_generated_from_the_header(pkg):
    """The committed Rust `-sys` source declares every prototype of the header, with the header's argument count,
    and is what the generator writes today."""
    import importlib.util
    import re
    spec = importlib.util.spec_from_file_location("rust_sys", pkg._lib.HERE / "rust_sys.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    assert mod.OUT.read_text() == mod.generate(), "run python triton-rs_b200/rust_sys.py"
    text = mod.OUT.read_text()
    protos = pkg.parse_header()
    for name, (_, args) in protos.items():
        m = re.search(r"pub fn " + name + r"\((.*?)\)", text, flags=re.S)
        assert m, name
        got = [a for a in m.group(1).split(",") if a.strip()]
        assert len(got) == len(args), name
    assert mod.rust_type("const b200k_half *") == "*const b200k_half"
    assert mod.rust_type("void **") == "*mut *mut c_void"
    assert mod.rust_type("struct b200k_comm **") == "*mut *mut b200k_comm"


def test_token_exchange_slot_size_formula(pkg):
    """fused_moe_a2a_slot_bytes = rows of every rank's pairs (256-byte rounded) + their id table; no device needed."""
    L = pkg.lib()
    for t_loc, h, k, world in [(64, 4096, 2, 8), (20, 256, 2, 2), (1, 64, 1, 1), (7, 128, 3, 4)]:
        slots = world * t_loc * k
        want = (slots * h * 2 + 255) // 256 * 256 + slots * 4
        assert L.call("fused_moe_a2a_slot_bytes", t_loc, h, k, world) == want
