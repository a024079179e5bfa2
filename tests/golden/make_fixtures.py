"""Regenerates the committed golden fixtures from the reference checkout.

    python tests/golden/make_fixtures.py /path/to/reference

Copies the reference's known-answer files for the block formats and the f32->f16 rounding,
and cuts a small subset out of its 10 MB quantiser round-trip fixture (the uncalibrated
Q4_K / Q5_K records only; 4 rows of 2560 and 2 rows of 10240 each).
Record formats: reference/dequant_ref.c:21-24 and reference/quant_ref.c:26-31.
"""
import os
import shutil
import struct
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def read_quant_records(path):
    b = open(path, "rb").read()
    o, recs = 0, []
    while o < len(b):
        typ, rows, k, im = struct.unpack_from("<IIII", b, o); o += 16
        x = b[o:o + 4 * rows * k]; o += 4 * rows * k
        imx = b""
        if im and path.endswith("_in.bin"):
            imx = b[o:o + 4 * k]; o += 4 * k
        recs.append((typ, rows, k, im, x, imx))
    return recs


def main(ref):
    shutil.copy(os.path.join(ref, "gguf/testdata/dequant_in.bin"), os.path.join(HERE, "dequant_in.bin"))
    shutil.copy(os.path.join(ref, "gguf/testdata/dequant_ref.bin"), os.path.join(HERE, "dequant_ref.bin"))
    shutil.copy(os.path.join(ref, "safetensors/testdata/f32_to_f16.txt"), os.path.join(HERE, "f32_to_f16.txt"))
    rin = read_quant_records(os.path.join(ref, "llm/testdata/quant_in.bin"))
    rref = read_quant_records(os.path.join(ref, "llm/testdata/quant_ref.bin"))
    assert len(rin) == len(rref)
    with open(os.path.join(HERE, "quant_subset_in.bin"), "wb") as fi, open(os.path.join(HERE, "quant_subset_ref.bin"), "wb") as fr:
        for a, b in zip(rin, rref):
            typ, rows, k, im = a[:4]
            if typ not in (12, 13) or im:
                continue
            keep = 4 if k <= 2560 else 2
            for f, rec in ((fi, a), (fr, b)):
                f.write(struct.pack("<IIII", typ, keep, k, 0))
                f.write(rec[4][:4 * keep * k])


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_fixtures.py <path of a checkout of the reference repository>")
    main(sys.argv[1])
