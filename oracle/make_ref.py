"""Place the reference's own model modules where the CPU timing leg can import them.

TEST / MEASUREMENT INFRASTRUCTURE ONLY.

    python oracle/make_ref.py --reference /path/to/pe_ablations

copies the reference's ``src/model/*.py`` (pure Python + torch + einops; no build step) into
``oracle/_ref/src/model/``.  That folder is ignored by git -- nothing of the reference is
committed -- but it is part of the working tree, so a machine that receives the tree without
the reference checkout (the GPU box) can still time the reference's real modules on its host
cores: ``oracle.cpu_baseline`` uses them when they are there (``kind = "reference"``) and
falls back to the restatement in ``oracle.pe_attention_oracle`` (``kind = "port"``) when not.
``__graft_entry__.build()`` runs this whenever the reference checkout is present.
"""

from __future__ import annotations

import argparse
import os
import shutil

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")


def make_ref(reference: str) -> str:
    src = os.path.join(reference, "src", "model")
    if not os.path.isdir(src):
        raise FileNotFoundError(f"{src} not found: --reference must point at a checkout of the reference project")
    dst = os.path.join(REF_DIR, "src", "model")
    os.makedirs(dst, exist_ok=True)
    for name in sorted(os.listdir(src)):
        if name.endswith(".py"):
            shutil.copyfile(os.path.join(src, name), os.path.join(dst, name))
    # the hot-path modules import nothing from src/model/kernels (a placeholder package)
    for pkg in (os.path.join(REF_DIR, "src"),):
        init = os.path.join(pkg, "__init__.py")
        if not os.path.exists(init):
            open(init, "w").close()
    return REF_DIR


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of a checkout of the reference project")
    print(make_ref(ap.parse_args().reference))
