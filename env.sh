#!/bin/bash
# Source this file (". env.sh") to use the framework from a checkout:
#   - puts the checkout first on PYTHONPATH and verifies that `import sga_b200` resolves to it
#     (an installed copy elsewhere on the path would otherwise shadow the tree being edited),
#   - locates nvcc and exports NVCC for the in-tree build,
#   - builds the native library when it is missing or stale.
# ". env.sh --check" only verifies and reports (exit status 1 on failure), it builds nothing.

_sga_env_main() {
    local root check=0
    root="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
    [ "${1:-}" = "--check" ] && check=1
    export SGA_B200_ROOT="$root"
    case ":${PYTHONPATH:-}:" in
        *":$root:"*) ;;
        *) export PYTHONPATH="$root${PYTHONPATH:+:$PYTHONPATH}" ;;
    esac
    local nvcc="${NVCC:-}"
    [ -z "$nvcc" ] && nvcc="$(command -v nvcc 2>/dev/null || true)"
    [ -z "$nvcc" ] && [ -x /usr/local/cuda/bin/nvcc ] && nvcc=/usr/local/cuda/bin/nvcc
    if [ -z "$nvcc" ]; then
        echo "env.sh: nvcc not found (set NVCC=/path/to/nvcc); the native library cannot be built" >&2
        return 1
    fi
    export NVCC="$nvcc"
    # anti-shadowing: the package that python imports must be the one under this checkout
    local where
    where="$(python3 -c 'import os, sga_b200; print(os.path.dirname(os.path.dirname(os.path.abspath(sga_b200.__file__))))' 2>/dev/null)"
    if [ "$where" != "$root" ]; then
        echo "env.sh: 'import sga_b200' resolves to '${where:-<import failed>}', not to $root" >&2
        return 1
    fi
    if [ "$check" = 1 ]; then
        echo "env.sh: ok (root $root, nvcc $nvcc)"
        return 0
    fi
    python3 "$root/sga_b200/csrc/build.py" > /dev/null || { echo "env.sh: native build failed" >&2; return 1; }
    return 0
}
_sga_env_main "$@"
_sga_env_rc=$?
unset -f _sga_env_main
(exit $_sga_env_rc)
