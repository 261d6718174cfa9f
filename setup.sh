#!/bin/bash
# Setup check: environment sanity (env.sh --check), toolchain against manifest.yaml, native build,
# and what the GPUs of this machine offer. Prints a report; exits 1 only when the framework cannot
# work here at all (no nvcc, import shadowed, build failure). Reads settings, changes none.
set -u
root="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
cd "$root"
echo "== sga_b200 setup check =="
if ! source "$root/env.sh" --check; then
    echo "FAIL: env.sh --check did not pass" >&2
    exit 1
fi
python3 - <<'PY'
import os, re, subprocess, sys
import yaml

root = os.environ["SGA_B200_ROOT"]
man = yaml.safe_load(open(os.path.join(root, "manifest.yaml")))
tc = man["toolchain"]
warn = 0


def note(kind, msg):
    global warn
    warn += kind == "WARN"
    print(f"{kind} {msg}")


out = subprocess.run([os.environ["NVCC"], "--version"], capture_output=True, text=True).stdout
m = re.search(r"release (\d+\.\d+)", out)
rel = m.group(1) if m else "?"
note("ok  " if rel == tc["cuda"] else "WARN", f"nvcc release {rel} (manifest {tc['cuda']})")
note("ok  " if sys.version_info[:2] >= tuple(int(x) for x in tc["python_min"].split(".")) else "WARN",
     f"python {sys.version.split()[0]} (manifest >= {tc['python_min']})")
try:
    import torch

    tv = tuple(int(x) for x in re.findall(r"\d+", torch.__version__)[:2])
    note("ok  " if tv >= tuple(int(x) for x in tc["torch_min"].split(".")) else "WARN",
         f"torch {torch.__version__} (manifest >= {tc['torch_min']})")
    if torch.cuda.is_available():
        n = torch.cuda.device_count()
        caps = {torch.cuda.get_device_capability(i) for i in range(n)}
        note("ok  " if caps == {(10, 0)} else "WARN", f"{n} GPU(s), compute capability {sorted(caps)} (kernels need 10.0)")
        if n > 1:
            bad = [(i, j) for i in range(n) for j in range(n) if i != j and not torch.cuda.can_device_access_peer(i, j)]
            note("ok  " if not bad else "WARN", f"peer access between all GPU pairs: {'yes' if not bad else bad[:4]}")
    else:
        note("WARN", "no GPU visible: CPU paths and the cross-compiled build only")
except Exception as e:  # noqa: BLE001
    note("WARN", f"torch not importable: {e}")
print(f"{warn} warning(s)")
PY
python3 "$root/sga_b200/csrc/build.py" > /dev/null || { echo "FAIL: native build" >&2; exit 1; }
echo "ok   native library built: $(ls "$root"/sga_b200/csrc/libsga_b200.so)"
