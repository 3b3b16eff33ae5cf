"""Generate tests/golden/hash64_reference.json by running the reference's own CPU helpers.

Run in a container that has the reference checkout:
    python tests/golden/make_golden.py /path/to/reference
It imports the reference's data_loader (numpy only) and records, for seeded
random byte states of the reference's native length 120, the values of
``hash_state_cpu`` and ``owner_rank_for_state``.  The inputs are regenerated
from the seed by the tests, so only seeds and outputs are stored.
"""

import json
import sys
from pathlib import Path

import numpy as np


def main() -> None:
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/reference")
    ref = Path(sys.argv[1]).resolve()
    sys.path.insert(0, str(ref))
    sys.dont_write_bytecode = True
    import data_loader  # type: ignore

    out = {"state_size": data_loader.STATE_SIZE, "cases": []}
    # case 0: the identity arrangement 0..119; cases 1..: seeded random bytes, two value ranges.
    states = [("arange", 0, np.arange(120, dtype=np.uint8))]
    for seed in range(1, 33):
        rng = np.random.default_rng(900000 + seed)
        hi = 120 if seed % 2 else 256
        states.append((f"uniform{hi}", 900000 + seed, rng.integers(0, hi, size=120, dtype=np.uint8)))
    for kind, seed, s in states:
        out["cases"].append({
            "kind": kind,
            "seed": seed,
            "hash64": int(data_loader.hash_state_cpu(s)),
            "owner_w2": int(data_loader.owner_rank_for_state(s, 2)),
            "owner_w3": int(data_loader.owner_rank_for_state(s, 3)),
            "owner_w8": int(data_loader.owner_rank_for_state(s, 8)),
        })
    dst = Path(__file__).resolve().parent / "hash64_reference.json"
    dst.write_text(json.dumps(out, indent=1))
    print(f"wrote {dst} ({len(out['cases'])} cases)")


if __name__ == "__main__":
    main()
