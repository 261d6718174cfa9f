#!/usr/bin/env python3
"""Audit a run yaml against the trainer's argument parser.

    python tests/audit_trainer_args.py dump  out.json                  every accepted flag (dest, default, choices, group)
    python tests/audit_trainer_args.py check run.yaml [out.json]       what the yaml turns into, and what the parser says
    python tests/audit_trainer_args.py diff-defaults old.json new.json compare two dumps flag by flag

``check`` reports two views, as the reference's ``tests/audit_megatron_args.py`` does for its parser:

  PRIMARY    the real launch pipeline (``launcher.run.load_config`` -> ``TrainBackend``): the flag list a node
             would run with, launcher-injected directories included. A refusal here decides the exit code.
  SECONDARY  the raw ``train.{system,model,data}`` leaves flattened directly: which of the authored keys are
             unknown to the parser, and which are accepted only for compatibility (this trainer has one
             choice for them, so they change nothing).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import tempfile

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def flag_table() -> dict:
    from sga_b200.runtime.trainer import build_parser

    table = {}
    parser = build_parser()
    for group in parser._action_groups:
        for a in group._group_actions:
            if not a.option_strings:
                continue
            table[a.option_strings[0]] = {"dest": a.dest, "default": a.default, "group": group.title,
                                          "choices": list(a.choices) if a.choices else None,
                                          "takes_value": a.nargs != 0}
    return table


def check(path: str) -> int:
    from sga_b200.launcher import backend as B
    from sga_b200.launcher.run import load_config, validate_task
    from sga_b200.launcher.utils import flatten_dict_to_args

    table = flag_table()
    rc = 0
    print(f"== PRIMARY: launch pipeline over {path}")
    try:
        cfg = load_config(path, [f"experiment.exp_dir={tempfile.mkdtemp(prefix='audit-exp-')}"])
        validate_task(cfg)
        args = B.TrainBackend(cfg).train_args
        print(f"   ok: {len(args)} tokens, {sum(1 for t in args if t.startswith('--'))} flags")
    except Exception as e:  # the pipeline's own refusal is the finding
        print(f"   REFUSED: {type(e).__name__}: {e}")
        rc = 1
    print("== SECONDARY: authored train.{system,model,data} leaves")
    import yaml

    raw = yaml.safe_load(open(path)) or {}
    flat = {}
    for section in ("system", "model", "data"):
        flat.update((raw.get("train") or {}).get(section) or {})
    tokens = flatten_dict_to_args(flat)
    flags = [t for t in tokens if t.startswith("--")]
    unknown = [f for f in flags if f not in table]
    compat = [f for f in flags if f in table and table[f]["group"] == "accepted for yaml compatibility"]
    print(f"   {len(flags)} flags; unknown to the parser: {unknown or 'none'}")
    print(f"   accepted for compatibility only: {compat or 'none'}")
    return rc or (1 if unknown else 0)


def diff_defaults(old_path: str, new_path: str) -> int:
    old, new = json.load(open(old_path)), json.load(open(new_path))
    for f in sorted(set(old) - set(new)):
        print(f"removed  {f}")
    for f in sorted(set(new) - set(old)):
        print(f"added    {f} (default {new[f]['default']!r})")
    for f in sorted(set(old) & set(new)):
        if old[f]["default"] != new[f]["default"] or old[f]["choices"] != new[f]["choices"]:
            print(f"changed  {f}: default {old[f]['default']!r} -> {new[f]['default']!r}, "
                  f"choices {old[f]['choices']} -> {new[f]['choices']}")
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    sub = ap.add_subparsers(dest="mode", required=True)
    sub.add_parser("dump").add_argument("out")
    c = sub.add_parser("check")
    c.add_argument("yaml")
    c.add_argument("out", nargs="?")
    d = sub.add_parser("diff-defaults")
    d.add_argument("old")
    d.add_argument("new")
    ns = ap.parse_args(argv)
    if ns.mode == "diff-defaults":
        return diff_defaults(ns.old, ns.new)
    rc = check(ns.yaml) if ns.mode == "check" else 0
    if ns.out:
        with open(ns.out, "w") as fh:
            json.dump(flag_table(), fh, indent=1, sort_keys=True, default=repr)
        print(f"flag table -> {ns.out}")
    return rc


if __name__ == "__main__":
    sys.exit(main())
