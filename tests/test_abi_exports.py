"""The C ABI library loads on a machine without a GPU and exports every symbol the header declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "pom_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pom_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = _declared_functions()
    for must in ("pom_gemm_bf16", "pom_ctx_gemm", "pom_gate_gemm", "pom_gate_bwd_gemm", "pom_poly_agg_fwd",
                 "pom_poly_agg_bwd", "pom_select_fwd", "pom_select_bwd", "pom_state_merge", "pom_reduce_partials"):
        assert must in names


def test_library_loads_and_exports_every_declared_symbol():
    from pom_b200 import _abi, _build

    _build.build()
    lib = _abi.lib()
    for name in _declared_functions():
        assert hasattr(lib, name), f"{name} declared in include/pom_b200.h but not exported"
        assert name in _abi._SIGNATURES, f"{name} has no ctypes signature"
    assert lib.pom_abi_version() == _abi.ABI_VERSION
    assert _abi.strerror(0) == "ok" and "degree" in _abi.strerror(-5)


def test_struct_sizes_match_the_c_compiler():
    """Guards the ctypes mirrors of the argument structs against drift from the header."""
    import subprocess
    import tempfile

    from pom_b200 import _abi

    structs = {"pom_rope": _abi.Rope, "pom_gemm_args": _abi.GemmArgs, "pom_ctx_args": _abi.CtxArgs,
               "pom_gate_args": _abi.GateArgs, "pom_gate_bwd_args": _abi.GateBwdArgs, "pom_agg_args": _abi.AggArgs,
               "pom_agg_bwd_args": _abi.AggBwdArgs, "pom_select_args": _abi.SelectArgs,
               "pom_select_bwd_args": _abi.SelectBwdArgs, "pom_select_heads_args": _abi.SelectHeadsArgs,
               "pom_layer_args": _abi.LayerArgs, "pom_heads_args": _abi.HeadsArgs, "pom_peer_comm": _abi.PeerComm, "pom_peer_xchg_args": _abi.PeerXchgArgs}
    src = '#include <stdio.h>\n#include "pom_b200.h"\nint main(void){' + "".join(
        f'printf("{n} %zu\\n", sizeof({n}));' for n in structs) + "return 0;}\n"
    with tempfile.TemporaryDirectory() as d:
        c = os.path.join(d, "s.c")
        open(c, "w").write(src)
        exe = os.path.join(d, "s")
        subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), c, "-o", exe], check=True)
        out = subprocess.run([exe], check=True, capture_output=True, text=True).stdout
    for line in out.strip().splitlines():
        name, size = line.split()
        assert ctypes.sizeof(structs[name]) == int(size), name


def test_missing_library_fails_loudly(monkeypatch):
    from pom_b200 import _abi

    monkeypatch.setattr(_abi, "_lib", None)
    monkeypatch.setattr(_abi, "LIB_PATH", "/nonexistent/libpom_b200.so")
    try:
        _abi.lib()
    except ImportError as e:
        assert "no CPU or PyTorch fallback" in str(e)
    else:
        raise AssertionError("expected ImportError")
