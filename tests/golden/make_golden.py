"""Makes tests/golden/reference_logits.json: logits of the reference's own CPU engine on two
tiny models, to anchor tests/plain_llama.py once; and tests/golden/reference_shapes.json: what
the reference's ``shapes`` command (cleanroom-transformer/src/main.c:528-536, src/shapes.c) prints
for the two configurations, to anchor the weight table.

Run from the repository root:  python tests/golden/make_golden.py /path/to/reference

It copies the reference's cleanroom-transformer/ to a temporary folder, builds it there
(``make CC=/usr/bin/gcc``), writes the two tiny model folders (weights from an integer hash,
so they are the same bits on every machine: tests/golden/golden_models.py), and runs the
reference's ``logits`` command (cleanroom-transformer/src/main.c:351-387) with the CPU
backend for several prefix lengths, with and without ``--split``.  Only token ids, a
sample of vocabulary ids and the resulting logits are stored.
"""
import json
import os
import shutil
import subprocess
import sys
import tempfile

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from golden_models import GOLDEN_MODELS, golden_tokens, write_golden_model  # noqa: E402


def main() -> None:
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/reference")
    ref = sys.argv[1]
    work = tempfile.mkdtemp(prefix="golden_")
    src = os.path.join(work, "ct")
    shutil.copytree(os.path.join(ref, "cleanroom-transformer"), src)
    subprocess.run(["make", "CC=/usr/bin/gcc"], cwd=src, check=True, stdout=subprocess.DEVNULL)
    exe = os.path.join(src, "build", "cleanroom-transformer")
    out = {"source": "reference CPU backend, `logits --backend cpu`", "cases": []}
    shapes = {}
    for name, spec in GOLDEN_MODELS.items():
        mdir = os.path.join(work, name)
        write_golden_model(mdir, spec)
        res = subprocess.run([exe, "shapes", "--model", mdir], check=True, capture_output=True, text=True)
        shapes[name] = json.loads(res.stdout)
        vocab = spec["config"]["vocab_size"]
        toks = golden_tokens(spec)
        ids = list(range(0, vocab, max(1, vocab // 24)))
        for n in spec["prefix_lengths"]:
            for split in (0, n // 2):
                cmd = [exe, "logits", "--model", mdir, "--backend", "cpu", "--max-tokens", "256",
                       "--tokens", " ".join(map(str, toks[:n])), "--ids", " ".join(map(str, ids))]
                if split:
                    cmd += ["--split", str(split)]
                res = subprocess.run(cmd, check=True, capture_output=True, text=True)
                vals = [float(x) for x in res.stdout.split()]
                assert len(vals) == len(ids)
                out["cases"].append({"model": name, "n_tokens": n, "split": split, "ids": ids, "logits": vals})
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_logits.json")
    with open(dst, "w") as f:
        json.dump(out, f)
    dst_shapes = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_shapes.json")
    with open(dst_shapes, "w") as f:
        f.write('{"source": "reference `shapes --model DIR`", "models": {\n')
        for i, (k, v) in enumerate(shapes.items()):
            f.write(f' "{k}": {json.dumps(v)}' + (",\n" if i + 1 < len(shapes) else "\n"))
        f.write("}}\n")
    shutil.rmtree(work)
    print("wrote", dst, len(out["cases"]), "cases;", dst_shapes)


if __name__ == "__main__":
    main()
