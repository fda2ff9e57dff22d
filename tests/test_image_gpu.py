"""Striped weight image on the GPU: scatter ingest of whole tensors and of per-rank expert slabs
through the C ABI gives back the exact bytes, and the device checksum equals the builder's."""
from __future__ import annotations

import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT / "oracle"))
import image_oracle  # noqa: E402


def _tensors():
    generator = torch.Generator().manual_seed(21)
    return {
        # expert tensors in checkpoint layout, 16 experts: per-expert slabs are 4 MiB and 2 MiB
        "layers.0.mlp.experts.gate_up_proj": torch.randn(16, 1024, 2048, generator=generator).to(torch.bfloat16),
        "layers.0.mlp.experts.down_proj": torch.randn(16, 2048, 512, generator=generator).to(torch.bfloat16),
        "layers.0.mlp.gate.weight": torch.randn(256, 2048, generator=generator).to(torch.bfloat16),
        "layers.0.post_attention_layernorm.weight": torch.randn(2048, generator=generator).to(torch.bfloat16),
        "odd.tail": torch.randn(3 * 4096 + 520, generator=generator).to(torch.bfloat16),      # not a multiple of 4096 bytes
    }


def test_ingest_returns_the_exact_bytes_and_checksum(package, tmp_path):
    device = torch.device("cuda", 0)
    image = package.StripedImage()
    tensors = _tensors()
    names = sorted(tensors)
    paths = (tmp_path / "lane0.bin", tmp_path / "lane1.bin")
    plan = image.build(*paths, names, tensors)
    destinations = [torch.zeros_like(tensors[name], device=device) for name in names]
    ranges = [(plan["aggregate_offset"][i], plan["payload_bytes"][i]) for i in range(len(names))]
    result = image.scatter_ingest(*paths, ranges, destinations, plan["lane_bytes"], chunk_bytes=1 << 20,
                                  expected=(plan["xor"], plan["sum"]))
    for name, got in zip(names, destinations):
        assert torch.equal(got.cpu(), tensors[name]), name
    assert result.bytes == sum(plan["payload_bytes"])
    assert (result.xor_value, result.sum_value) == (plan["xor"], plan["sum"])
    assert (result.xor_value, result.sum_value) == image_oracle.checksum(
        [tensors[name].view(torch.int16).numpy() for name in names])
    # a wrong expectation fails closed
    with pytest.raises(package.AimaMoeError):
        image.scatter_ingest(*paths, ranges, destinations, plan["lane_bytes"], expected=(plan["xor"] ^ 1, plan["sum"]))


@pytest.mark.parametrize("world", [2, 4, 8])
def test_ingest_of_per_rank_expert_slabs(package, tmp_path, world):
    device = torch.device("cuda", 0)
    image = package.StripedImage()
    tensors = _tensors()
    names = sorted(tensors)
    paths = (tmp_path / "lane0.bin", tmp_path / "lane1.bin")
    plan = image.build(*paths, names, tensors)
    expert_names = [n for n in names if "experts" in n]
    per_rank = 16 // world
    for rank in (0, world - 1):
        ranges, destinations, want = [], [], []
        for name in expert_names:
            i = names.index(name)
            slab = tensors[name][rank * per_rank:(rank + 1) * per_rank]
            slab_bytes = slab.numel() * 2
            ranges.append((plan["aggregate_offset"][i] + rank * slab_bytes, slab_bytes))
            destinations.append(torch.zeros_like(slab, device=device))
            want.append(slab)
        result = image.scatter_ingest(*paths, ranges, destinations, plan["lane_bytes"], chunk_bytes=4 << 20)
        for got, expected in zip(destinations, want):
            assert torch.equal(got.cpu(), expected)
        assert (result.xor_value, result.sum_value) == image_oracle.checksum(
            [w.contiguous().view(torch.int16).numpy() for w in want])


def test_ingest_argument_checks(package, tmp_path):
    device = torch.device("cuda", 0)
    image = package.StripedImage()
    tensors = _tensors()
    names = sorted(tensors)
    paths = (tmp_path / "lane0.bin", tmp_path / "lane1.bin")
    plan = image.build(*paths, names, tensors)
    destination = torch.zeros(4096, dtype=torch.bfloat16, device=device)
    with pytest.raises(package.AimaMoeError):      # offset not a multiple of 4096
        image.scatter_ingest(*paths, [(8, 8192)], [destination], plan["lane_bytes"])
    with pytest.raises(package.AimaMoeError):      # range runs past the end of its lane
        image.scatter_ingest(*paths, [(plan["lane_bytes"][0] - 4096, 8192)], [destination], plan["lane_bytes"])
    with pytest.raises(package.AimaMoeError):      # host destination
        image.scatter_ingest(*paths, [(0, 8192)], [torch.zeros(4096, dtype=torch.bfloat16)], plan["lane_bytes"])
