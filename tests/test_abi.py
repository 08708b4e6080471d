"""Host-side checks that need no GPU: the C-ABI library loads, exports every symbol the
public header declares, and fails loudly (never falls back) without a device."""
import ctypes as C

import pytest


def test_library_exports_every_declared_symbol(cm):
    syms = cm.declared_symbols()
    assert len(syms) >= 45
    missing = [s for s in syms if not hasattr(cm.lib(), s)]
    assert missing == []
    # every declared symbol has a ctypes signature in the binding
    unbound = [s for s in syms if s not in cm.lib()._signatures]
    assert unbound == []
    assert cm.lib().cmld_version().startswith(b"camelid_b200")


def test_row_size_helpers(cm):
    # codes + f32 scales per 32 + i16 sums per 16, each rounded to 16 bytes
    assert cm.act_row_bytes(4096) == 4096 + 512 + 512
    assert cm.act_row_bytes(64) == 64 + 16 + 16


def test_no_device_is_an_error_not_a_fallback(cm):
    if cm.device_count() > 0:
        pytest.skip("a CUDA device is present")
    cfg = cm.EngineConfig(n_layers=1, n_heads=2, n_kv_heads=1, head_dim=32, hidden=64, ffn_dim=128, max_pos=16, vocab=96)
    with pytest.raises(cm.CmldError) as ei:
        cm.ResidentDecode(cfg)
    assert ei.value.code == 5 and "no CPU path" in ei.value.message


def test_config_validation_messages(cm):
    from camelid_b200._lib import Config, check

    bad = cm.EngineConfig(n_layers=1, n_heads=3, n_kv_heads=2, head_dim=32, hidden=96, ffn_dim=128, max_pos=16, vocab=96)
    h = C.c_void_p()
    c = bad.to_c()
    rc = cm.lib().cmld_engine_create(C.byref(c), C.byref(h))
    assert rc == 2 and b"n_kv_heads" in cm.lib().cmld_last_error()
    assert cm.lib().cmld_engine_create(None, C.byref(h)) == 1
    # null handles are rejected, not dereferenced
    assert cm.lib().cmld_engine_set_filled(None, 0) == 1
    assert cm.lib().cmld_engine_weights_ready(None) == 0
    assert cm.lib().cmld_weight_wire_bytes(None) == 0


def test_synthetic_model_byte_counts(cm):
    from camelid_b200 import synth

    # bytes read per decode token, against the reference's tensor-table figure for the 1B
    # Q8_0 model (1.3133 GB, qa/evidence-bundles/sirocco-phase0-roofline-20260712/README.md)
    c = synth.engine_config("llama-1b", 512)
    assert abs(synth.weight_bytes_per_token(c, "q8_0") / 1e9 - 1.3133) < 1e-3
    assert synth.kv_bytes_per_position(c) == 32 * 1024
    c = synth.engine_config("llama-8b", 8192)
    assert abs(synth.weight_bytes_per_token(c, "q4_k_m") / 1e9 - 4.8769) < 1e-3
    assert synth.kv_bytes_per_position(c) == 128 * 1024


def test_header_compiles_as_cxx_and_links_against_the_static_archive(cm, tmp_path):
    """include/camelid_b200.h is compiled, not only mirrored by hand in the ctypes binding: a small C++ program
    includes it, links libcamelid_b200.a (+ the CUDA runtime) and exercises cmld_engine_create / cmld_last_error."""
    import shutil
    import subprocess
    from pathlib import Path

    from camelid_b200 import build

    root = Path(__file__).resolve().parent.parent
    build.build()
    assert build.STATIC_LIB.exists()
    cuda = Path(shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc").resolve().parent.parent
    if not (cuda / "lib64" / "libcudart_static.a").exists():
        pytest.skip("the static CUDA runtime is not installed")
    exe = tmp_path / "abi_link_check"
    cmd = ["g++", "-std=c++17", "-Wall", "-Werror", "-I", str(root / "include"), str(root / "tests" / "abi_link_check.cpp"),
           str(build.STATIC_LIB), "-L", str(cuda / "lib64"), "-lcudart_static", "-ldl", "-lpthread", "-lrt", "-o", str(exe)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    run = subprocess.run([str(exe)], capture_output=True, text=True)
    assert run.returncode == 0 and run.stdout.startswith("ok camelid_b200"), (run.returncode, run.stdout, run.stderr)
