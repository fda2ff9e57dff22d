"""CPU tests of the drop-in boundary: the shared library loads without a GPU, exports every
symbol include/aima_moe.h declares, and its argument checks fail closed."""
from __future__ import annotations

import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
HEADER = ROOT / "include" / "aima_moe.h"


def _declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(aima_moe_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree(package, built_library):
    declared = _declared_functions()
    bound = sorted(name for name, _, _ in package.provider.EXPORTS)
    assert declared == bound


def test_library_exports_every_declared_symbol(package, built_library):
    library = ctypes.CDLL(str(built_library), mode=ctypes.RTLD_LOCAL)
    for name in _declared_functions():
        assert hasattr(library, name), name
    lib = package.load_library()
    assert lib.aima_moe_abi_version() >> 16 == 1


def test_header_is_plain_c_and_cxx(tmp_path):
    """The boundary is a C ABI: the header must compile alone as C99 and as C++17 (a cgo, JNI or dlopen host
    includes nothing else), and a C host must link against the library by name."""
    import shutil
    import subprocess

    if shutil.which("gcc") is None or shutil.which("g++") is None:
        pytest.skip("no host compiler")
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Wextra", "-Werror", "-pedantic", "-fsyntax-only", "-x", "c", str(HEADER)],
                   check=True)
    subprocess.run(["g++", "-std=c++17", "-Wall", "-Wextra", "-Werror", "-fsyntax-only", "-x", "c++", str(HEADER)],
                   check=True)
    host = tmp_path / "host.c"
    host.write_text('#include "aima_moe.h"\nint main(void) { return (int)(aima_moe_abi_version() >> 16) == 1 ? 0 : 1; }\n')
    subprocess.run(["gcc", "-std=c99", "-I", str(HEADER.parent), "-c", str(host), "-o", str(tmp_path / "host.o")], check=True)


def test_the_documented_cxx_loader_compiles_and_resolves_every_symbol(built_library, tmp_path):
    """The dlopen / dlsym loader printed in INTEGRATION.md, compiled as it stands and run against the library."""
    import shutil
    import subprocess

    if shutil.which("g++") is None:
        pytest.skip("no host compiler")
    text = (ROOT / "INTEGRATION.md").read_text()
    block = text.split("```cpp\n", 1)[1].split("```", 1)[0]
    assert "load_moe_provider" in block
    source = tmp_path / "loader.cpp"
    source.write_text(block + """
int main(int argc, char** argv) {
  if (argc < 2) return 2;
  MoeProviderApi api = load_moe_provider(argv[1]);
  return (api.prepare && api.bind_layer && api.prefill_launch && api.decode_launch && api.sync_metrics &&
          api.release && api.last_error) ? 0 : 1;
}
""")
    binary = tmp_path / "loader"
    subprocess.run(["g++", "-std=c++17", "-Wall", "-Werror", "-I", str(HEADER.parent), str(source), "-o", str(binary), "-ldl"],
                   check=True)
    subprocess.run([str(binary), str(built_library)], check=True)


def test_struct_sizes_match_the_header(package):
    p = package.provider
    assert ctypes.sizeof(p.Config) == 12 * 4
    assert ctypes.sizeof(p.LayerWeights) == 8 + 8 * 16
    assert ctypes.sizeof(p.DebugViews) == 8 + 12 * 8
    assert ctypes.sizeof(p.Metrics) == 8 + 5 * 8 + 8 + 16 + 24


def test_argument_checks_fail_closed_without_a_device(package, built_library):
    import torch

    p = package.provider
    lib = package.load_library()
    size = ctypes.c_uint64()
    good = p.Config(ctypes.sizeof(p.Config), 2048, 256, 8, 512, 512, 40, 8192, 1, 0, 1e-6, 0)
    assert lib.aima_moe_query_workspace(ctypes.byref(good), ctypes.byref(size)) == 0
    assert size.value > 8192 * 8 * 2048 * 2 * 2          # gathered rows + expert outputs
    bad_shape = p.Config(ctypes.sizeof(p.Config), 4096, 256, 8, 512, 512, 40, 0, 1, 0, 1e-6, 0)
    assert lib.aima_moe_query_workspace(ctypes.byref(bad_shape), ctypes.byref(size)) == -2
    bad_size = p.Config(4, 2048, 256, 8, 512, 512, 40, 0, 1, 0, 1e-6, 0)
    assert lib.aima_moe_query_workspace(ctypes.byref(bad_size), ctypes.byref(size)) == -1
    assert b"size mismatch" in lib.aima_moe_last_error_string()
    bad_world = p.Config(ctypes.sizeof(p.Config), 2048, 256, 8, 512, 512, 40, 0, 3, 0, 1e-6, 0)
    assert lib.aima_moe_query_workspace(ctypes.byref(bad_world), ctypes.byref(size)) == -1
    bad_rank = p.Config(ctypes.sizeof(p.Config), 2048, 256, 8, 512, 512, 40, 0, 2, 2, 1e-6, 0)
    assert lib.aima_moe_query_workspace(ctypes.byref(bad_rank), ctypes.byref(size)) == -1
    # null handle paths never touch a device
    assert lib.aima_moe_decode_launch(None, 0, None, None, None, None) == -1
    assert lib.aima_moe_prefill_launch(None, 0, None, None, None, 1, None, None) == -1
    assert lib.aima_moe_release(None) == 0
    if not torch.cuda.is_available():
        handle = ctypes.c_void_p()
        status = lib.aima_moe_prepare(ctypes.byref(good), ctypes.byref(handle))
        assert status == -7 and not handle.value        # AIMA_MOE_ERR_NO_DEVICE, no fallback
        with pytest.raises(RuntimeError):
            package.MoeProvider(layers=1)


def test_synthetic_layers_are_reproducible(synth):
    import torch

    a = synth.expert_gate_up(1234, 3, 17)
    b = synth.expert_gate_up(1234, 3, 17)
    c = synth.expert_gate_up(1234, 3, 18)
    assert torch.equal(a, b) and not torch.equal(a, c)
    assert a.shape == (1024, 2048) and a.dtype == torch.bfloat16
    assert abs(float(a.float().std()) - 0.02) < 5e-4
    bias = synth.zipf_router_bias(1)
    assert bias.shape == (256,) and abs(float(bias.mean())) < 1e-6
    x = synth.activations(1, 64)
    assert abs(float(x.float().std()) - 1.0) < 0.02


def test_lm_head_and_image_argument_checks_need_no_device(package, built_library):
    lib = package.load_library()
    handle = ctypes.c_void_p()
    assert lib.aima_moe_lm_head_build(None, 10, ctypes.byref(handle), None) == -1 and not handle.value
    assert lib.aima_moe_lm_head_launch(None, None, None, None) == -1
    assert lib.aima_moe_lm_head_release(None) == 0
    count = ctypes.c_uint64(7)
    assert lib.aima_moe_safetensors_index(b"/nonexistent/file.safetensors", None, 0, ctypes.byref(count)) == -1
    assert count.value == 0 and b"cannot open" in lib.aima_moe_last_error_string()
    assert lib.aima_moe_image_plan(None, None, 0, None, None, None, None) == -1
    x, s = ctypes.c_uint64(0), ctypes.c_uint64(0)
    assert lib.aima_moe_image_checksum_host(ctypes.c_char_p(b"1234567"), 7, ctypes.byref(x), ctypes.byref(s)) == -1
    p = package.provider
    assert ctypes.sizeof(p.LmHeadResult) == 24 and ctypes.sizeof(p.ImageIngestResult) == 40
    assert ctypes.sizeof(p.SafetensorsEntry) == 200 + 8 + 8 + 32 + 16
