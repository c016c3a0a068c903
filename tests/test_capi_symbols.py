"""CPU checks of the drop-in boundary: header, binding table and exported symbols agree."""
import re
import subprocess
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
BIN = ROOT / "cuda-c-diffusion_b200" / "build" / "bin"  # built by cuda-c-diffusion_b200/csrc/host/Makefile
HEADER = ROOT / "include" / "b200_layer_kernels.h"


def _header_prototypes():
    src = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return re.findall(r"\n\s*(?:void|int|long long|const char\*)\s+((?:launch_|b200_)\w+)\s*\(([^;]*?)\)\s*;", src)


def _code(arg):
    arg = arg.strip()
    if arg in ("void", ""):
        return ""
    if "cudaStream_t" in arg:
        return "s"
    if any(k in arg for k in ("B200ParamUpdate", "B200WeightDesc", "B200WeightGradDesc", "B200PeerDests", "B200CopyItem", "char*")):
        return "h"
    if "*" in arg:
        return "p"
    if arg.startswith("long long"):
        return "q"
    if arg.startswith("float"):
        return "f"
    if arg.startswith("int") or arg.startswith("b200_act_t"):
        return "i"
    raise ValueError(arg)


def test_header_declares_the_42_reference_launchers(capi):
    names = [n for n, _ in _header_prototypes()]
    assert len(capi.REFERENCE_LAUNCHERS) == 42
    for n in capi.REFERENCE_LAUNCHERS:
        assert n in names, f"{n} missing from include/b200_layer_kernels.h"
        assert n.startswith("launch_")


def test_binding_table_matches_header(capi):
    protos = _header_prototypes()
    assert {n for n, _ in protos} == set(capi.SIGNATURES)
    for name, args in protos:
        assert "".join(_code(a) for a in args.split(",")) == capi.SIGNATURES[name], name


def test_every_header_prototype_cites_the_reference_or_says_it_has_none():
    text = HEADER.read_text()
    # each reference launcher is preceded (within the same group) by a nn.h citation
    assert text.count("nn.h:") >= 30
    assert "No counterpart in the reference" in text and "no counterpart in the reference" in text


def test_library_loads_and_exports_every_symbol(capi):
    lib = capi.load()  # raises ImportError on a missing symbol or missing build
    assert lib.b200_version().startswith(b"b200-layer-kernels")
    out = subprocess.run(["nm", "-D", "--defined-only", str(capi.LIB_PATH)], capture_output=True, text=True, check=True)
    exported = {ln.split()[-1] for ln in out.stdout.splitlines() if " T " in ln}
    for name in capi.SIGNATURES:
        assert name in exported, name


def test_reference_host_modules_link_against_our_library():
    """build/bin/gradcheck_b200 is the reference's unmodified gradcheck.c and host
    modules linked with this library in place of its kernels.o."""
    exe = BIN / "gradcheck_b200"
    if not exe.exists():
        import pytest
        pytest.skip("host programs not built here")
    out = subprocess.run(["nm", "-D", "--undefined-only", str(exe)], capture_output=True, text=True, check=True)
    needed = {ln.split()[-1] for ln in out.stdout.splitlines() if "launch_" in ln}
    assert needed, "gradcheck_b200 should import launch_* from the shared library"
    lib = subprocess.run(["nm", "-D", "--defined-only", str(ROOT / "cuda-c-diffusion_b200" / "libb200_layer_kernels.so")],
                         capture_output=True, text=True, check=True).stdout
    for n in needed:
        assert f" T {n}" in lib, n


def test_error_mode_records_instead_of_exiting(capi):
    import ctypes
    lib = capi.load()
    lib.b200_set_error_mode(1)
    lib.b200_clear_error()
    # C not divisible by G is rejected on the host before anything touches a device
    lib.launch_groupnorm_forward(None, None, None, None, None, None, 1, 4, 6, 4, ctypes.c_float(1e-5), None)
    assert lib.b200_error_count() == 1
    buf = ctypes.create_string_buffer(512)
    lib.b200_last_error(ctypes.cast(buf, ctypes.c_void_p), 512)
    assert b"divisible" in buf.value
    lib.launch_sinusoidal(None, None, 2, 7, ctypes.c_float(9.2), None)
    assert lib.b200_error_count() == 2
    lib.b200_clear_error()
    lib.b200_set_error_mode(0)
