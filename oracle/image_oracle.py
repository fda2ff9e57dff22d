"""CPU restatement (numpy) of the striped weight image's two integer algorithms.  TEST INFRASTRUCTURE ONLY.

* layout: "deterministic LPT by descending aligned bytes then tensor name; assign to the lower-total lane
  with lane0 winning ties", extents aligned to 4096 bytes
  (engine/production-striped-image-manifest.json, layout.algorithm) -- pinned against that manifest's 693
  entries through tests/golden/striped_layout.json.
* checksum: XOR and wrapping 64-bit SUM over the payload's uint64 words
  (benchmarks/shape-lab/native/src/striped_image_builder.cpp:137-147).
"""
from __future__ import annotations

import numpy as np

ALIGNMENT = 4096


def aligned(nbytes: int) -> int:
    return (nbytes + ALIGNMENT - 1) // ALIGNMENT * ALIGNMENT


def lpt_plan(names: list[str], payload_bytes: list[int]) -> dict:
    order = sorted(range(len(names)), key=lambda i: (-aligned(payload_bytes[i]), names[i].encode()))
    totals = [0, 0]
    lane = [0] * len(names)
    lane_offset = [0] * len(names)
    for i in order:
        chosen = 0 if totals[0] <= totals[1] else 1
        lane[i] = chosen
        lane_offset[i] = totals[chosen]
        totals[chosen] += aligned(payload_bytes[i])
    aggregate = [(0 if lane[i] == 0 else totals[0]) + lane_offset[i] for i in range(len(names))]
    return {"lane": lane, "lane_offset": lane_offset, "aggregate_offset": aggregate, "lane_bytes": totals}


def checksum(buffers: list[np.ndarray]) -> tuple[int, int]:
    xor_value = np.uint64(0)
    sum_value = np.uint64(0)
    with np.errstate(over="ignore"):
        for buffer in buffers:
            words = np.frombuffer(np.ascontiguousarray(buffer).tobytes(), dtype=np.uint64)
            xor_value ^= np.bitwise_xor.reduce(words) if words.size else np.uint64(0)
            sum_value = np.uint64((int(sum_value) + int(words.sum(dtype=np.uint64))) % (1 << 64))
    return int(xor_value), int(sum_value)
