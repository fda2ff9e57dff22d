"""Builds oracle/_ref/libmoe_ref.so: the reference's OWN scalar kernels for the MoE path, compiled
for the host.  Test infrastructure -- nothing in the product may load it.

The kernels are not copied into this repository.  At build time their definitions are cut out of
the reference checkout (its location: AIMA_REFERENCE_ROOT in the environment) into oracle/_ref/ (ignored by
git), and compiled with g++ against a small stand-in for the HIP device constructs they use
(oracle/ref_shim/) and the launcher in oracle/ref_driver.cpp.  Taken, by name:

  native/src/native_moe_prefill.hip.cpp   shared_silu_multiply_batched_kernel, shared_sigmoid_scale_batched_kernel,
                                          router_topk8_softmax_256_kernel, moe_align_block32_256_kernel,
                                          expert_silu_multiply_kernel, moe_sum8_kernel
  native/src/native_pointwise.hip.cpp     pytorch_rounded_rsqrtf, bf16_add_pair_kernel, prefill_rmsnorm_2048_kernel,
                                          prefill_add_rmsnorm_2048_kernel, shared_activation_kernel, shared_gate_kernel
  native/src/native_lm_head.hip.cpp       quantize_lm_head_rowwise_kernel

Two builds: libmoe_ref.so with -ffp-contract=off (the source as written) and libmoe_ref_fma.so with
-ffp-contract=fast -mfma (the contraction licence hipcc takes by default).  They can differ only where
a product is not exact in FP32 -- on this path that is the LM-head residual; squares and products of
BF16 values are exact, so RMSNorm, SwiGLU and the routing are the same in both.

Without the reference checkout (e.g. on a GPU box) this script does nothing and the prebuilt
libraries, if present, are used as they are.
"""
from __future__ import annotations

import os
import re
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
REFERENCE = Path(os.environ.get("AIMA_REFERENCE_ROOT", "/root/reference"))

WANTED = [
    ("native/src/native_moe_prefill.hip.cpp", "ref_moe",
     ["kHidden", "kExperts", "kTopK", "kSharedIntermediate", "kExpertGateUp", "kMoeBlock", "kThreads"],
     ["shared_silu_multiply_batched_kernel", "shared_sigmoid_scale_batched_kernel",
      "router_topk8_softmax_256_kernel", "moe_align_block32_256_kernel", "expert_silu_multiply_kernel",
      "moe_sum8_kernel"]),
    ("native/src/native_pointwise.hip.cpp", "ref_pointwise",
     ["kThreads", "kHidden", "kSharedIntermediate"],
     ["pytorch_rounded_rsqrtf", "bf16_add_pair_kernel", "prefill_rmsnorm_2048_kernel",
      "prefill_add_rmsnorm_2048_kernel", "shared_activation_kernel", "shared_gate_kernel"]),
    ("native/src/native_lm_head.hip.cpp", "ref_lm_head",
     ["kRows", "kColumns", "kThreads", "kResidualSafetyUlps"],
     ["quantize_lm_head_rowwise_kernel"]),
]


def cut_constant(text: str, name: str) -> str:
    match = re.search(r"^constexpr\s+[\w:\s\*]+?\b%s\s*=[^;]*;" % re.escape(name), text, re.M)
    if match is None:
        raise RuntimeError(f"constant {name} not found in the reference source")
    return match.group(0)


def cut_function(text: str, name: str) -> str:
    match = re.search(r"^(?:__global__|__device__)[^;{}]*?\b%s\s*\(" % re.escape(name), text, re.M)
    if match is None:
        raise RuntimeError(f"function {name} not found in the reference source")
    open_brace = text.index("{", match.end())
    depth, position = 0, open_brace
    while True:
        character = text[position]
        if character == "{":
            depth += 1
        elif character == "}":
            depth -= 1
            if depth == 0:
                break
        position += 1
    return text[match.start():position + 1]


def extract() -> Path:
    OUT.mkdir(exist_ok=True)
    pieces = ["// GENERATED from the reference checkout by oracle/build_ref.py -- not tracked, do not edit.\n"]
    for relative, namespace, constants, functions in WANTED:
        text = (REFERENCE / relative).read_text()
        pieces.append(f"// ---- {relative} ----\nnamespace {namespace} {{\n")
        pieces += [cut_constant(text, name) + "\n" for name in constants]
        pieces += [cut_function(text, name) + "\n\n" for name in functions]
        pieces.append(f"}}  // namespace {namespace}\n\n")
    target = OUT / "ref_extracted.inc"
    target.write_text("".join(pieces))
    return target


def compile_library(name: str, contraction: list[str]) -> Path:
    target = OUT / name
    command = ["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-fno-fast-math", *contraction,
               "-I", str(HERE / "ref_shim"), "-I", str(OUT), str(HERE / "ref_driver.cpp"), "-o", str(target)]
    result = subprocess.run(command, capture_output=True, text=True)
    if result.returncode != 0:
        sys.stderr.write(result.stdout + result.stderr)
        raise RuntimeError(f"g++ failed building {name}")
    return target


sys.path.insert(0, str(HERE))


def build(force: bool = False) -> list[Path]:
    """Returns the built libraries; an empty list when the reference checkout is absent."""
    libraries = [OUT / "libmoe_ref.so", OUT / "libmoe_ref_fma.so"]
    if not (REFERENCE / "native/src/native_moe_prefill.hip.cpp").is_file():
        return [path for path in libraries if path.is_file()]
    sources = [HERE / "ref_driver.cpp", Path(__file__), *(HERE / "ref_shim" / "hip").glob("*.h")]
    newest = max(path.stat().st_mtime for path in sources)
    if not force and all(path.is_file() and path.stat().st_mtime > newest for path in libraries):
        return libraries
    extract()
    import reference_torch        # the torch functions of the same checkout, for the benchmark's reference arm

    reference_torch.write_extracted()
    import reference_triton       # its Triton decode kernels, run under Triton's interpreter by the golden generator

    reference_triton.write_extracted()
    compile_library("libmoe_ref.so", ["-ffp-contract=off"])
    compile_library("libmoe_ref_fma.so", ["-ffp-contract=fast", "-mfma"])
    return libraries


if __name__ == "__main__":
    built = build(force="--force" in sys.argv)
    print("\n".join(str(path) for path in built) if built else "reference checkout absent: nothing built")
