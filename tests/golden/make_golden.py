r"""Turns what the reference itself produced on a B200 into the committed fixtures.

Pipeline (the first two steps need the reference sources and a GPU; their output is what this script reads):
  1. python oracle/build_ref.py
         builds the reference unmodified (oracle/_ref/vdnn_ref) and oracle/ref/ref_harness.cu linked against
         the reference's own Layer class (oracle/_ref/ref_harness), both on cuDNN / cuBLAS
  2. on a GPU box, with NVIDIA_TF32_OVERRIDE=0 and VDNN_POOL_BYTES=60000000000:
         oracle/_ref/ref_harness <raw_dir>
         oracle/_ref/vdnn_ref {MODEL} {POLICY} {ALGO} | grep -E "WorkSpaceSize|\[Fwd\]|\[Bwd\]" > <runs_dir>/{MODEL}_{POLICY}_{ALGO}.log
  3. python tests/golden/make_golden.py <raw_dir> <runs_dir>
         writes tests/golden/ref_layers.npz (+ ref_layers.json) and tests/golden/ref_memory.json
  4. for the layers at benchmark size:   oracle/_ref/ref_harness <big_dir> big    (same environment), then
     python tests/golden/make_golden.py --big <big_dir>
         writes tests/golden/ref_big.npz (+ ref_big.json): per tensor 4096 evenly strided samples, and in the json its
         element count, stride, sum, sum of squares and largest magnitude over the whole tensor

ref_layers: outputs of the reference's Layer::forward / Layer::backward for every layer type on seeded
inputs (inputs are regenerated in the tests from the same counter-based generator).
ref_memory: the per-layer "Memory Usage" figures and workspace sizes printed by the reference program
(network.cu:1069-1074, 1098-1103, 1129-1134, 1176-1181; layer.cu:480-484).
"""
import json
import os
import re
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def pack_layers(raw_dir):
    manifest = json.load(open(os.path.join(raw_dir, "manifest.json")))
    arrays = {}
    for f in sorted(os.listdir(raw_dir)):
        if f.endswith(".bin"):
            arrays[f[:-4]] = np.fromfile(os.path.join(raw_dir, f), dtype="<f4")
    np.savez_compressed(os.path.join(HERE, "ref_layers.npz"), **arrays)
    json.dump(manifest, open(os.path.join(HERE, "ref_layers.json"), "w"), indent=1)
    print(f"ref_layers: {len(arrays)} tensors, {sum(a.size for a in arrays.values())} floats")


def pack_memory(runs_dir):
    out = {}
    for f in sorted(os.listdir(runs_dir)):
        if not f.endswith(".log"):
            continue
        m = re.match(r"(ALEXNET|OVERFEAT|VGG16_64|VGG16_128)_(BASELINE|VDNN_NONE|VDNN_ALL|VDNN_CONV)_(VDNN_\w+_ALGO)\.log", f)
        ws, fwd, bwd = {}, [], []
        for line in open(os.path.join(runs_dir, f)):
            w = re.match(r"CONV Layer (\d+) (fwd|bwdData|bwdFilter)WorkSpaceSize: (\d+)", line)
            if w:
                ws.setdefault(int(w.group(1)), {})[w.group(2)] = int(w.group(3))
            u = re.match(r"\[(Fwd|Bwd)\] Layer (\d+), Free Memory: (\d+), Total Memory: (\d+), Memory Usage: (\d+)", line)
            if u:
                rec = [int(u.group(2)), int(u.group(4)) - int(u.group(3)), int(u.group(5))]   # layer, used, printed usage
                (fwd if u.group(1) == "Fwd" else bwd).append(rec)
        out["/".join(m.groups())] = {"workspace": {str(k): [v["fwd"], v["bwdData"], v["bwdFilter"]] for k, v in sorted(ws.items())},
                                      "fwd": fwd, "bwd": bwd}
    json.dump(out, open(os.path.join(HERE, "ref_memory.json"), "w"))
    print(f"ref_memory: {len(out)} runs")


def pack_big(raw_dir):
    manifest = json.load(open(os.path.join(raw_dir, "manifest.json")))
    arrays = {t["name"]: np.fromfile(os.path.join(raw_dir, t["name"] + ".bin"), dtype="<f4") for t in manifest["tensors"]}
    for t in manifest["tensors"]:
        assert arrays[t["name"]].size == t["samples"], t
    np.savez_compressed(os.path.join(HERE, "ref_big.npz"), **arrays)
    json.dump(manifest, open(os.path.join(HERE, "ref_big.json"), "w"), indent=1)
    print(f"ref_big: {len(arrays)} tensors reduced to {sum(a.size for a in arrays.values())} samples")


if __name__ == "__main__":
    if sys.argv[1] == "--big":
        pack_big(sys.argv[2])
    else:
        pack_layers(sys.argv[1])
        pack_memory(sys.argv[2])
