"""CPU: the Rust `extern "C"` crate against the header, mechanically (no Rust toolchain exists here, so the crate
is never compiled): every declaration of include/b200_moe.h must appear in rust/b200-moe-sys/src/lib.rs with the
same number of arguments, every struct with the same field names in the same order, every constant with the same
value; and every `sys::` function the safe crate calls must exist with the argument count it is called with."""
import importlib.util
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SYS = os.path.join(ROOT, "rust", "b200-moe-sys")


def _gen():
    spec = importlib.util.spec_from_file_location("gen_bindings", os.path.join(SYS, "gen_bindings.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _rust_items(text):
    fns = {}
    for m in re.finditer(r"pub fn (b200_\w+)\((.*?)\)(?: -> [^;]+)?;", text, flags=re.S):
        args = m.group(2).strip()
        depth, n = 0, (1 if args else 0)
        for ch in args:
            depth += ch in "(<"
            depth -= ch in ")>"
            n += ch == "," and depth == 0
        fns[m.group(1)] = n
    structs = {m.group(1): re.findall(r"pub (\w+):", m.group(2))
               for m in re.finditer(r"pub struct (\w+) \{(.*?)\n\}", text, flags=re.S)}
    consts = {m.group(1): int(m.group(2)) for m in re.finditer(r"pub const (B200_\w+): c_int = (\d+);", text)}
    return fns, structs, consts


def test_sys_crate_matches_header():
    gen = _gen()
    api = gen.parse_header()
    text = open(os.path.join(SYS, "src", "lib.rs")).read()
    assert text == gen.generate(api), "rust/b200-moe-sys/src/lib.rs is stale: run gen_bindings.py"
    fns, structs, consts = _rust_items(text)
    assert set(fns) == set(api["functions"]) and len(fns) >= 45
    for name, (_ret, args) in api["functions"].items():
        assert fns[name] == len(args), name
    for name, fields in api["structs"].items():
        assert structs[name] == [f for _t, f in fields], name
    for name in api["opaque"]:
        assert name in structs
    assert consts == {**api["defines"], **api["enums"]}


def test_header_matches_ctypes_table():
    """The same header parse against the Python binding's table: one more independent reading of the ABI."""
    import __graft_entry__ as ge
    pkg = ge.load_package()
    from mlx_rs_b200 import _lib
    api = _gen().parse_header()
    assert set(api["functions"]) == set(_lib.EXPORTS)
    for name, (_ret, args) in api["functions"].items():
        assert len(_lib.EXPORTS[name][1]) == len(args), name
    assert pkg is not None


def test_safe_crate_calls_existing_functions():
    api = _gen().parse_header()
    src = os.path.join(ROOT, "rust", "b200-moe", "src")
    called = 0
    for f in os.listdir(src):
        text = open(os.path.join(src, f)).read()
        for m in re.finditer(r"sys::(b200_\w+)\(", text):
            name = m.group(1)
            assert name in api["functions"], f"{f}: {name} is not in the header"
            # count the call's top-level arguments
            i, depth, n, seen = m.end(), 1, 0, False
            while depth:
                ch = text[i]
                depth += ch in "([{"
                depth -= ch in ")]}"
                if depth >= 1 and not ch.isspace():
                    seen = True
                n += ch == "," and depth == 1
                i += 1
            n += seen
            assert n == len(api["functions"][name][1]), f"{f}: {name} called with {n} arguments"
            called += 1
    assert called >= 20
