"""Build the bf16 screening copy of a trace.

``python -m sga_b200.trace_convert --src SRC --dst DST [--from-step A] [--to-step B] [--overwrite]``

Every ``step_*_g.pt`` payload whose step lies in ``[A, B)`` is rounded to bf16
per tensor (round-to-nearest: bit-identical to a run that dumped bf16
directly; tensors that are not fp32 pass through), the state files of that
range are copied verbatim, and the catalog is copied with ``g_dtype: bf16`` so
that the copy describes itself. The source is never written. A destination
that already holds files is refused unless ``--overwrite`` is given, and then
every trace file in it is removed first: the destination is a trace, and a
leftover step file would make a reader see the union of two step sets. A
source that is already bf16 converts to an identical copy, with a warning.
Files are written to a temporary name and renamed.

CLI surface and rules: ``sga/trace_convert.py:35-143``.
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


def convert_trace(src: str, dst: str, overwrite: bool = False, from_step=None, to_step=None, log=None) -> dict:
    """Returns ``{"g_files", "state_files", "src_bytes", "dst_bytes", "dst"}`` (bytes over the g files)."""
    cat_path = os.path.join(src, "catalog.pt")
    if not os.path.isfile(cat_path):
        raise ValueError(f"no catalog.pt in --src {src}")
    if os.path.realpath(src) == os.path.realpath(dst):
        raise ValueError("--dst must differ from --src (the source trace is never modified in place)")
    if from_step is not None and to_step is not None and to_step <= from_step:
        raise ValueError(f"--to-step must be > --from-step, got {from_step}..{to_step}")
    held = os.listdir(dst) if os.path.isdir(dst) else []
    if held and not overwrite:
        raise ValueError(f"--dst {dst} exists and is not empty (use --overwrite to reuse)")
    for name in held:
        if name == "catalog.pt" or _G.match(name) or _S.match(name):
            os.unlink(os.path.join(dst, name))
    os.makedirs(dst, exist_ok=True)

    cat = torch.load(cat_path, map_location="cpu", weights_only=False)
    if str(cat.get("g_dtype", "fp32")) == "bf16":
        say = log if log is not None else (lambda m, **kw: print(m, file=sys.stderr, **kw))
        say("WARNING: source catalog g_dtype is already bf16: this conversion rounds nothing", flush=True)
    cat = dict(cat)
    cat["g_dtype"] = "bf16"
    _atomic_save(cat, os.path.join(dst, "catalog.pt"))

    def wanted(step: int) -> bool:
        return (from_step is None or step >= from_step) and (to_step is None or step < to_step)

    n_g = n_s = src_bytes = dst_bytes = 0
    for name in sorted(os.listdir(src)):
        sp, dp = os.path.join(src, name), os.path.join(dst, name)
        mg, ms = _G.match(name), _S.match(name)
        if mg and wanted(int(mg.group(1))):
            blob = torch.load(sp, map_location="cpu", weights_only=False)
            blob["payload"] = {k: (v.to(torch.bfloat16) if torch.is_tensor(v) and v.dtype == torch.float32 else v)
                               for k, v in blob["payload"].items()}
            _atomic_save(blob, dp)
            n_g += 1
            src_bytes += os.path.getsize(sp)
            dst_bytes += os.path.getsize(dp)
            if log is not None and n_g % 100 == 0:
                log(f"g {n_g} files converted (last step {int(mg.group(1))})", flush=True)
        elif ms and wanted(int(ms.group(1))):
            shutil.copy2(sp, dp + ".tmp")
            os.replace(dp + ".tmp", dp)
            n_s += 1
    return {"g_files": n_g, "state_files": n_s, "src_bytes": src_bytes, "dst_bytes": dst_bytes, "dst": dst}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="build a bf16 screening copy of a trace (g payloads fp32->bf16; states "
                                             "verbatim; catalog verbatim except the g_dtype=bf16 tag; source untouched)")
    ap.add_argument("--src", required=True, help="source trace directory")
    ap.add_argument("--dst", required=True, help="destination directory")
    ap.add_argument("--from-step", type=int, default=None, help="convert g/state files from this step (inclusive)")
    ap.add_argument("--to-step", type=int, default=None, help="up to this step (exclusive); default: whole trace")
    ap.add_argument("--overwrite", action="store_true", help="allow writing into a non-empty --dst")
    ns = ap.parse_args(argv)
    res = convert_trace(ns.src, ns.dst, ns.overwrite, ns.from_step, ns.to_step, log=print)
    print(f"done: {res['g_files']} g files converted ({res['src_bytes'] / 1e9:.2f} GB -> "
          f"{res['dst_bytes'] / 1e9:.2f} GB), {res['state_files']} state files copied")
    return 0


if __name__ == "__main__":
    sys.exit(main())
