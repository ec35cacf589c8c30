"""The OCaml externals ship as source (no OCaml toolchain on the image), so
drift between the C header, the stubs and the `external` declarations is
caught here on the CPU: the stubs are compiled with -fsyntax-only against a
stand-in for the runtime's headers (tests/caml_standin), which checks every
call into the library against include/oxgpu_b200.h; and every `external` is
matched with a stub of the same arity, with a bytecode/native pair where OCaml
requires one (more than five arguments)."""
import os
import re
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
STUBS = os.path.join(ROOT, "ocaml", "oxgpu_b200_stubs.c")
ML = os.path.join(ROOT, "ocaml", "oxgpu_b200.ml")


def test_stubs_compile_against_the_header():
    cmd = ["gcc", "-std=c11", "-fsyntax-only", "-Wall", "-Wextra", "-Werror=incompatible-pointer-types",
           "-Werror=int-conversion", "-Werror=implicit-function-declaration", "-Werror=return-type",
           "-I", os.path.join(ROOT, "tests", "caml_standin"), STUBS]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    assert proc.returncode == 0, proc.stderr


def _stub_arities():
    """name -> number of `value` parameters, or 'byte' for (value *argv, int argn)."""
    text = open(STUBS).read()
    # expand the two-entry-point macro the buffer stubs are generated with
    for name in re.findall(r"^BUFFER_STUB\((\w+),", text, flags=re.M):
        text += f"\nCAMLprim value {name}(" + ", ".join(f"value a{i}" for i in range(11)) + ") {}\n"
        text += f"\nCAMLprim value {name}_byte(value *argv, int argn) {{}}\n"
    out = {}
    for name, params in re.findall(r"CAMLprim value (\w+)\(([^)]*)\)", text):
        if name == "NAME" or name.startswith("NAME"):
            continue
        params = " ".join(params.split())
        if params.startswith("value *argv"):
            out[name] = "byte"
        else:
            out[name] = len([p for p in params.split(",") if p.strip().startswith("value ")])
    return out


def _externals():
    """(ocaml name, arity, [stub names]) for every `external` declaration."""
    text = re.sub(r"\(\*.*?\*\)", "", open(ML).read(), flags=re.S)
    out = []
    for name, ty, stubs in re.findall(r"external\s+(\w+)\s*:\s*(.*?)\s*=\s*((?:\"\w+\"\s*)+)", text, flags=re.S):
        depth, arrows, i = 0, 0, 0
        while i < len(ty):                       # top-level arrows only: (a * b) array, ('a, 'b, c) t ...
            ch = ty[i]
            if ch == "(":
                depth += 1
            elif ch == ")":
                depth -= 1
            elif ty.startswith("->", i) and depth == 0:
                arrows += 1
                i += 1
            i += 1
        out.append((name, arrows, re.findall(r"\"(\w+)\"", stubs)))
    return out


def test_every_external_has_a_stub_of_its_arity():
    stubs = _stub_arities()
    ext = _externals()
    assert len(ext) >= 30
    for name, arity, names in ext:
        if arity > 5:
            assert len(names) == 2, f"{name}: more than five arguments needs a bytecode and a native stub"
            byte, native = names
            assert stubs.get(byte) == "byte", f"{name}: {byte} must take (value *argv, int argn)"
        else:
            assert len(names) == 1, name
            native = names[0]
        assert stubs.get(native) == arity, f"{name}: stub {native} takes {stubs.get(native)} values, external has {arity}"


def test_the_surface_covers_the_path():
    names = {n for n, _, _ in _externals()}
    for must in ("gemm_tmap", "gemm_bf16", "gemm_tf32", "gemm_exact", "encode_tmap_2d", "transpose",
                 "fill_uniform", "fill_normal", "gemm_bf16_host", "gemm_bf16_host_checked", "device_status",
                 "mg_create", "mg_gemm_bf16", "mg_gemm_bf16_host", "mg_sync", "mg_destroy", "mg_alloc",
                 "mg_copy_string_to_device", "mg_column_partition", "choose_config_raw", "kernel_binding"):
        assert must in names, must
