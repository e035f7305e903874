"""Reads the layer-shape tables of the reference's end-to-end timing mode
(include/timing/shapes_e2e.h: ResNet18/34/152, VGG16/19, DarkNet19/53 as rows of
c, ih, iw, kn, kw, kh, p, s) and writes them as data to fastertnn_b200/model_tables.json.

    python tests/golden/make_model_tables.py <reference checkout>

Only numbers are taken over: each model becomes a list of [C, H, W, KN, KH, KW, P, S] rows in
the order the reference runs them (src/timing_layers.c:186-202 feeds every layer's output
to the next layer)."""
import json
import re
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]


def parse(header: str):
    models = {}
    for m in re.finditer(r"static\s+int\s+shapes_(\w+)\s*\[[^\]]*\]\s*\[[^\]]*\]\s*=\s*\{(.*?)\};", header, flags=re.S):
        name, body = m.group(1), re.sub(r"//[^\n]*", "", m.group(2))
        rows = []
        for r in re.finditer(r"\{([^{}]*)\}", body):
            v = [int(t) for t in r.group(1).replace(" ", "").split(",") if t]
            assert len(v) == 8, (name, v)
            c, ih, iw, kn, kw, kh, p, s = v
            rows.append([c, ih, iw, kn, kh, kw, p, s])
        models[name] = rows
    return models


def main():
    ref = Path(sys.argv[1])
    models = parse((ref / "include" / "timing" / "shapes_e2e.h").read_text())
    out = {"source": "include/timing/shapes_e2e.h of fpgasystems/FasterTNN", "columns": ["C", "H", "W", "KN", "KH", "KW", "P", "S"],
           "batch": 8, "models": models}
    (ROOT / "fastertnn_b200" / "model_tables.json").write_text(json.dumps(out, indent=None, separators=(",", ":")) + "\n")
    for k, v in models.items():
        print(k, len(v))


if __name__ == "__main__":
    main()
