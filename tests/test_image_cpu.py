"""Striped weight image, the parts that need no GPU: the layout planner of the C ABI reproduces the
reference's own manifest (693 tensors: lane, offset in the lane, offset in the aggregate, lane totals),
agrees with the numpy oracle, and the builder writes exactly the planned bytes."""
from __future__ import annotations

import json
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT / "oracle"))
import image_oracle  # noqa: E402

GOLDEN = json.loads((ROOT / "tests" / "golden" / "striped_layout.json").read_text())


def test_planner_reproduces_the_reference_manifest(package, built_library):
    image = package.StripedImage()
    entries = GOLDEN["entries"]
    names = [e[0] for e in entries]
    payload = [e[1] for e in entries]
    # the order in which tensors are presented must not matter: shuffle deterministically
    order = np.random.default_rng(7).permutation(len(entries))
    plan = image.plan([names[i] for i in order], [payload[i] for i in order])
    for position, i in enumerate(order):
        _, _, aligned, lane, lane_offset, aggregate = entries[i]
        assert plan["lane"][position] == lane
        assert plan["lane_offset"][position] == lane_offset
        assert plan["aggregate_offset"][position] == aggregate
        assert image_oracle.aligned(payload[i]) == aligned
    assert plan["lane_bytes"] == GOLDEN["lane_bytes"]
    assert sum(plan["lane_bytes"]) == GOLDEN["aligned_bytes"]
    want = image_oracle.lpt_plan(names, payload)
    assert want["lane_bytes"] == GOLDEN["lane_bytes"]
    assert want["lane"] == [e[3] for e in entries] and want["lane_offset"] == [e[4] for e in entries]


def test_checksum_matches_the_oracle(package, built_library):
    image = package.StripedImage()
    generator = torch.Generator().manual_seed(5)
    a = torch.randint(-2**62, 2**62, (4099,), generator=generator, dtype=torch.int64)
    b = torch.randn(1024, 8, generator=generator).to(torch.bfloat16)
    got = image.checksum(b, image.checksum(a))
    assert got == image_oracle.checksum([a.numpy(), b.view(torch.int16).numpy()])
    assert image.checksum(torch.zeros(8, dtype=torch.int64)) == (0, 0)


def test_builder_writes_the_planned_bytes(package, built_library, tmp_path):
    image = package.StripedImage()
    generator = torch.Generator().manual_seed(9)
    tensors = {
        "layers.0.experts.gate_up_proj": torch.randn(4, 64, 128, generator=generator).to(torch.bfloat16),
        "layers.0.experts.down_proj": torch.randn(4, 128, 32, generator=generator).to(torch.bfloat16),
        "layers.0.gate.weight": torch.randn(256, 100, generator=generator).to(torch.bfloat16),   # not a multiple of 4096
        "norm.weight": torch.randn(2048, generator=generator).to(torch.bfloat16),
    }
    names = sorted(tensors)
    plan = image.build(tmp_path / "lane0.bin", tmp_path / "lane1.bin", names, tensors)
    files = [np.fromfile(tmp_path / "lane0.bin", dtype=np.uint8), np.fromfile(tmp_path / "lane1.bin", dtype=np.uint8)]
    assert [f.size for f in files] == plan["lane_bytes"]
    covered = [np.zeros(f.size, dtype=bool) for f in files]
    for i, name in enumerate(names):
        raw = tensors[name].view(torch.int16).numpy().tobytes()
        lane, offset = plan["lane"][i], plan["lane_offset"][i]
        assert offset % 4096 == 0
        assert files[lane][offset:offset + len(raw)].tobytes() == raw
        covered[lane][offset:offset + len(raw)] = True
    for lane in range(2):
        assert not files[lane][~covered[lane]].any()            # padding is zero
    assert (plan["xor"], plan["sum"]) == image_oracle.checksum([tensors[n].view(torch.int16).numpy() for n in names])


def _write_safetensors(path, tensors: dict, metadata: dict | None = None) -> dict:
    """Writes the safetensors container by hand (8-byte header length, JSON header, data section)."""
    import struct

    header, blobs, cursor = {}, [], 0
    if metadata is not None:
        header["__metadata__"] = metadata
    for name, tensor in tensors.items():
        raw = tensor.contiguous().view(torch.int16).numpy().tobytes()
        header[name] = {"dtype": "BF16", "shape": list(tensor.shape), "data_offsets": [cursor, cursor + len(raw)]}
        blobs.append(raw)
        cursor += len(raw)
    text = json.dumps(header, separators=(",", ":")).encode()
    text += b" " * ((8 - len(text) % 8) % 8)
    with open(path, "wb") as handle:
        handle.write(struct.pack("<Q", len(text)))
        handle.write(text)
        for raw in blobs:
            handle.write(raw)
    return {name: (8 + len(text) + spec["data_offsets"][0], 8 + len(text) + spec["data_offsets"][1])
            for name, spec in header.items() if name != "__metadata__"}


def test_safetensors_index_and_build_from_shards(package, built_library, tmp_path):
    image = package.StripedImage()
    generator = torch.Generator().manual_seed(13)
    shard_a = {
        "model.language_model.layers.0.mlp.experts.gate_up_proj": torch.randn(4, 64, 128, generator=generator).to(torch.bfloat16),
        "model.language_model.layers.0.mlp.gate.weight": torch.randn(256, 128, generator=generator).to(torch.bfloat16),
    }
    shard_b = {
        "model.language_model.layers.0.mlp.experts.down_proj": torch.randn(4, 128, 32, generator=generator).to(torch.bfloat16),
        'odd "name"\\with escapes': torch.randn(3, 5, 8, generator=generator).to(torch.bfloat16),
    }
    want_a = _write_safetensors(tmp_path / "a.safetensors", shard_a, {"format": "pt", "nested": {"k": [1, 2, {"x": None}]}})
    want_b = _write_safetensors(tmp_path / "b.safetensors", shard_b)
    sources, truth = [], {}
    for path, tensors, want in ((tmp_path / "a.safetensors", shard_a, want_a), (tmp_path / "b.safetensors", shard_b, want_b)):
        index = image.safetensors_index(path)
        assert sorted(e["name"] for e in index) == sorted(tensors)
        for entry in index:
            assert entry["dtype"] == "BF16" and entry["shape"] == list(tensors[entry["name"]].shape)
            assert (entry["begin"], entry["end"]) == want[entry["name"]]
            sources.append({**entry, "path": path})
            truth[entry["name"]] = tensors[entry["name"]]
    plan = image.build_from_files(tmp_path / "lane0.bin", tmp_path / "lane1.bin", sources)
    files = [np.fromfile(tmp_path / "lane0.bin", dtype=np.uint8), np.fromfile(tmp_path / "lane1.bin", dtype=np.uint8)]
    for i, name in enumerate(plan["names"]):
        raw = truth[name].contiguous().view(torch.int16).numpy().tobytes()
        offset = plan["lane_offset"][i]
        assert files[plan["lane"][i]][offset:offset + len(raw)].tobytes() == raw
    assert (plan["xor"], plan["sum"]) == image_oracle.checksum(
        [truth[name].contiguous().view(torch.int16).numpy() for name in plan["names"]])
    # a truncated file and a malformed header fail closed
    (tmp_path / "bad.safetensors").write_bytes(b"\x10\x00\x00\x00\x00\x00\x00\x00{\"a\":")
    import pytest
    with pytest.raises(package.AimaMoeError):
        image.safetensors_index(tmp_path / "bad.safetensors")
