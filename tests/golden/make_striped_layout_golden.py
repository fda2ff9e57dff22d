"""Extracts the layout facts of the reference's striped weight image into tests/golden/striped_layout.json.

Source: engine/production-striped-image-manifest.json of the reference checkout (schema
aima-amd395-qwen36/striped-image-manifest/v1): per tensor its name, payload bytes, aligned bytes, lane,
offset inside the lane file and offset in the two-lane aggregate, plus the lane totals.  The planner in
this repository must reproduce lane and offsets from names and sizes alone.  Run once where the
reference checkout is available:

    python tests/golden/make_striped_layout_golden.py /path/to/reference
"""
from __future__ import annotations

import json
import sys
from pathlib import Path


def main() -> None:
    reference = Path(sys.argv[1])
    manifest = json.loads((reference / "engine" / "production-striped-image-manifest.json").read_text())
    out = {
        "alignment_bytes": manifest["layout"]["alignment_bytes"],
        "aligned_bytes": manifest["layout"]["aligned_bytes"],
        "payload_bytes": manifest["layout"]["payload_bytes"],
        "lane_bytes": [lane["image_bytes"] for lane in manifest["lanes"]],
        "entries": [[e["name"], e["payload_bytes"], e["aligned_bytes"], e["lane"], e["lane_offset_bytes"],
                     e["aggregate_offset_bytes"]] for e in manifest["entries"]],
    }
    target = Path(__file__).resolve().parent / "striped_layout.json"
    target.write_text(json.dumps(out, separators=(",", ":")))
    print(f"wrote {target} ({len(out['entries'])} entries)")


if __name__ == "__main__":
    main()
