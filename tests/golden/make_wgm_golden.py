"""Generate tests/golden/wgm_map_460x64_wgm8.npz from the reference's stored output.

Input : <reference>/src/gemm/ref/res -- the committed output of the reference's remap
        checker src/gemm/ref/map.cpp (nwg0 = 460, nwg1 = 64, WORK_GROUP_MAPPING = 8),
        29 440 lines "(wg0,wg1)--->(wg0', wg1') in original map".
Output: a compressed array file holding the four integer columns in file order and the
        SHA-256 of the text it was parsed from.

Run once where the reference tree is mounted:
    python tests/golden/make_wgm_golden.py <root of the reference tree>
"""
import hashlib
import pathlib
import re
import sys

import numpy as np


def main() -> None:
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    ref_root = pathlib.Path(sys.argv[1])
    text = (ref_root / "src/gemm/ref/res").read_bytes()
    pat = re.compile(rb"\((\d+),(\d+)\)--->\s*\((\d+),\s*(\d+)\) in original map")
    rows = [tuple(int(g) for g in m.groups()) for m in pat.finditer(text)]
    arr = np.asarray(rows, dtype=np.uint16)
    assert arr.shape == (460 * 64, 4), arr.shape
    out = pathlib.Path(__file__).with_name("wgm_map_460x64_wgm8.npz")
    np.savez_compressed(
        out,
        pairs=arr,
        nwg0=np.uint32(460),
        nwg1=np.uint32(64),
        wgm=np.uint32(8),
        source_sha256=np.bytes_(hashlib.sha256(text).hexdigest().encode()),
    )
    print(out, arr.shape, out.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
