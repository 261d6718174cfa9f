"""Convert an fp32 trace directory into its bf16 screening copy.

State files are copied verbatim, every ``step_*_g.pt`` payload is rounded to
bf16 per tensor (round-to-nearest, bit-identical to a run that dumped bf16
directly), and the catalog gets ``g_dtype: bf16``. Writes are atomic
(temporary file + rename); an existing destination must already be a bf16
copy of the same catalog. ``python -m sga_b200.trace_convert SRC DST``.
Reference: ``sga/trace_convert.py:35-143``.
"""
from __future__ import annotations

import argparse
import os
import re
import shutil
import sys

import torch

_G = re.compile(r"^step_(\d{6})_g\.pt$")
_S = re.compile(r"^step_(\d{6})_state\.pt$")


def _atomic_save(obj, path):
    tmp = f"{path}.tmp.{os.getpid()}.0"
    torch.save(obj, tmp)
    os.replace(tmp, path)


def convert_trace(src: str, dst: str, overwrite: bool = False) -> dict:
    cat_path = os.path.join(src, "catalog.pt")
    if not os.path.exists(cat_path):
        raise FileNotFoundError(f"{src} is not a trace directory (no catalog.pt)")
    cat = torch.load(cat_path, weights_only=False)
    if cat.get("g_dtype", "fp32") != "fp32":
        raise ValueError(f"source trace already stores g as {cat.get('g_dtype')}")
    os.makedirs(dst, exist_ok=True)
    dst_cat = os.path.join(dst, "catalog.pt")
    if os.path.exists(dst_cat) and not overwrite:
        old = torch.load(dst_cat, weights_only=False)
        if old.get("g_dtype") != "bf16" or old.get("catalog") != cat.get("catalog"):
            raise ValueError(f"{dst} holds a different trace; refusing to mix")
    out = dict(cat)
    out["g_dtype"] = "bf16"
    _atomic_save(out, dst_cat)
    n_g = n_s = 0
    for name in sorted(os.listdir(src)):
        sp, dp = os.path.join(src, name), os.path.join(dst, name)
        if _S.match(name):
            if not os.path.exists(dp) or overwrite:
                shutil.copyfile(sp, dp + ".tmp")
                os.replace(dp + ".tmp", dp)
            n_s += 1
        elif _G.match(name):
            if os.path.exists(dp) and not overwrite:
                n_g += 1
                continue
            blob = torch.load(sp, weights_only=False)
            blob["payload"] = {k: v.to(torch.bfloat16) for k, v in blob["payload"].items()}
            _atomic_save(blob, dp)
            n_g += 1
    return {"g_files": n_g, "state_files": n_s, "dst": dst}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("src")
    ap.add_argument("dst")
    ap.add_argument("--overwrite", action="store_true")
    ns = ap.parse_args(argv)
    res = convert_trace(ns.src, ns.dst, ns.overwrite)
    print(f"[trace_convert] {res['g_files']} g files, {res['state_files']} state files -> {res['dst']}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
