"""The Rust bindings under ``rust/`` against the C header, without a Rust toolchain.

``rust/ratchet-cuda-sys/src/lib.rs`` declares every entry point of ``include/ratchet_cuda.h`` for Rust;
``rust/ratchet-cuda/src/*.rs`` is the safe layer ratchet-core's ``Device::CUDA`` arms call.  Nothing here
compiles Rust, so the two files are read as text: every function of the header must appear in the
``extern "C"`` block with the same number of arguments, corresponding types and return type; every
``#[repr(C)]`` struct must list the header's fields in order with corresponding types; every enumerator
must have a constant of the same value; and every ``sys::rcu_*`` call of the safe layer must name a
declared function and pass as many arguments as it takes.
"""
import pathlib
import re

ROOT = pathlib.Path(__file__).resolve().parents[1]
HEADER = ROOT / "include" / "ratchet_cuda.h"
SYS = ROOT / "rust" / "ratchet-cuda-sys" / "src" / "lib.rs"
SAFE = ROOT / "rust" / "ratchet-cuda" / "src"

C_SCALARS = {"int32_t": "i32", "uint32_t": "u32", "uint64_t": "u64", "int64_t": "i64", "uint16_t": "u16", "uint8_t": "u8",
             "int": "c_int", "float": "f32", "double": "f64", "void": "c_void", "char": "c_char", "rcu_status": "rcu_status"}


def strip_c(text):
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"//[^\n]*", "", text)
    return re.sub(r"^\s*#.*$", "", text, flags=re.M)


def c_type(decl, named=True):
    """'const rcu_tensor* const* inputs' -> (canonical type, name).  Canonical: (pointee type name, constness of
    each pointer level from the innermost outwards, array length or None)."""
    decl = decl.strip()
    arr = re.match(r"^(.*?)([A-Za-z_]\w*)\s*\[\s*(\w*)\s*\]$", decl)
    n_arr = None
    if arr:
        decl, n_arr = f"{arr.group(1).strip()} {arr.group(2)}", arr.group(3)
    toks = decl.replace("*", " * ").split()
    name = toks.pop() if named else None
    i, const = 0, False
    if toks[i] == "const":
        const, i = True, i + 1
    base = toks[i]
    i += 1
    if i < len(toks) and toks[i] == "const":
        const, i = True, i + 1
    levels = []
    while i < len(toks):
        assert toks[i] == "*", decl
        i += 1
        levels.append("const" if const else "mut")
        const = False
        if i < len(toks) and toks[i] == "const":
            const, i = True, i + 1
    return (C_SCALARS.get(base, base), tuple(levels), n_arr), name


def rust_type(t):
    t = t.strip()
    levels = []
    while True:
        m = re.match(r"^\*(const|mut)\s+(.*)$", t)
        if not m:
            break
        levels.append(m.group(1))
        t = m.group(2).strip()
    n_arr = None
    m = re.match(r"^\[\s*(\w+)\s*;\s*(\w+)\s*\]$", t)
    if m:
        t, n_arr = m.group(1), m.group(2)
    # Rust writes the outermost pointer first, C the innermost: reverse to C's order
    return (t, tuple(reversed(levels)), n_arr)


def header_functions():
    text = strip_c(HEADER.read_text())
    out = {}
    for ret, name, params in re.findall(r"([A-Za-z_][\w \*]*?)\b(rcu_[a-z0-9_]+)\s*\(([^;{}()]*)\)\s*;", text, flags=re.S):
        ps = [p for p in (x.strip() for x in params.replace("\n", " ").split(",")) if p and p != "void"]
        args = []
        for p in ps:
            ty, nm = c_type(p)
            if ty[2] is not None:                      # an array parameter is a pointer to its element
                ty = (ty[0], ty[1] + ("mut",), None)
            args.append((nm, ty))
        ret = ret.strip()
        out[name] = (None if ret == "void" else c_type(ret, named=False)[0], args)
    return out


def rust_functions():
    text = re.sub(r"//[^\n]*", "", SYS.read_text())
    block = re.search(r'extern\s+"C"\s*\{(.*?)\n\}', text, flags=re.S).group(1)
    out = {}
    for name, params, ret in re.findall(r"pub fn (rcu_[a-z0-9_]+)\s*\(([^)]*)\)\s*(?:->\s*([^;]+))?;", block, flags=re.S):
        args = []
        for p in (x.strip() for x in params.split(",")):
            if p:
                nm, ty = p.split(":", 1)
                args.append((nm.strip(), rust_type(ty)))
        out[name] = (rust_type(ret) if ret else None, args)
    return out


def test_every_header_function_is_declared_for_rust_with_matching_signature():
    c, r = header_functions(), rust_functions()
    assert len(c) > 90, "the header parser lost most declarations"
    assert sorted(set(c) - set(r)) == [], "declared in the header, missing from the extern block"
    assert sorted(set(r) - set(c)) == [], "declared for Rust, absent from the header"
    assert list(c) == list(r), "the extern block follows the header's order"
    for name, (c_ret, c_args) in c.items():
        r_ret, r_args = r[name]
        assert len(c_args) == len(r_args), f"{name}: {len(c_args)} arguments in C, {len(r_args)} in Rust"
        assert c_ret == r_ret, f"{name}: returns {c_ret} in C, {r_ret} in Rust"
        for (c_nm, c_ty), (r_nm, r_ty) in zip(c_args, r_args):
            assert c_ty == r_ty, f"{name}({c_nm}): {c_ty} in C, {r_ty} in Rust"
            assert c_nm == r_nm, f"{name}: argument {c_nm} is called {r_nm} in Rust"


def header_structs():
    text = strip_c(HEADER.read_text())
    out = {}
    for body, name in re.findall(r"typedef\s+struct(?:\s+\w+)?\s*\{([^}]*)\}\s*(rcu_\w+)\s*;", text, flags=re.S):
        fields = []
        for line in body.split(";"):
            line = " ".join(line.split())
            if not line:
                continue
            # "uint32_t a, b" declares two fields of one type
            first, *more = [x.strip() for x in line.split(",")]
            ty, nm = c_type(first)
            fields.append((nm, ty))
            for m in more:
                fields.append((m, ty))
        out[name] = fields
    return out


def rust_structs():
    text = re.sub(r"//[^\n]*", "", SYS.read_text())
    out = {}
    for attrs, name, body in re.findall(r"((?:#\[[^\]]*\]\s*)+)pub struct (rcu_\w+)\s*\{([^}]*)\}", text, flags=re.S):
        assert "repr(C)" in attrs, f"{name} must be #[repr(C)]"
        fields = []
        for f in body.split(",\n"):
            f = f.strip().rstrip(",")
            if f:
                nm, ty = f.split(":", 1)
                fields.append((nm.replace("pub", "").strip(), rust_type(ty)))
        out[name] = fields
    return out


def test_structs_have_the_headers_fields_in_order():
    c, r = header_structs(), rust_structs()
    assert {"rcu_tensor", "rcu_decoder_config", "rcu_decoder_layer"} <= set(c)
    consts = dict(re.findall(r"pub const (\w+): usize = (\d+);", SYS.read_text()))
    for name, c_fields in c.items():
        assert name in r, f"struct {name} is not declared for Rust"
        r_fields = r[name]
        assert [n for n, _ in c_fields] == [n for n, _ in r_fields], name
        for (nm, c_ty), (_, r_ty) in zip(c_fields, r_fields):
            c_n, r_n = c_ty[2], r_ty[2]
            if r_n in consts:                          # RCU_MAX_RANK on both sides, or its value
                r_n = r_n if c_n == r_n else consts[r_n]
            c_n = consts.get(c_n, c_n) if c_n != r_n else c_n
            assert (c_ty[0], c_ty[1], c_n) == (r_ty[0], r_ty[1], r_n), f"{name}.{nm}: {c_ty} in C, {r_ty} in Rust"


def test_enumerators_have_constants_of_the_same_value():
    text = strip_c(HEADER.read_text())
    rust = dict(re.findall(r"pub const (RCU_\w+): [\w:]+ = (\d+);", SYS.read_text()))
    seen = 0
    for body in re.findall(r"enum(?:\s+\w+)?\s*\{([^}]*)\}", text, flags=re.S):
        value = -1
        for item in body.split(","):
            item = item.strip()
            if not item:
                continue
            if "=" in item:
                nm, v = (x.strip() for x in item.split("="))
                value = int(v, 0)
            else:
                nm, value = item, value + 1
            assert nm in rust, f"{nm} has no Rust constant"
            assert int(rust[nm]) == value, f"{nm} = {value} in C, {rust[nm]} in Rust"
            seen += 1
    for nm, v in re.findall(r"#define\s+(RCU_\w+)\s+(\d+)u?\b", HEADER.read_text()):
        assert nm in rust and int(rust[nm]) == int(v), f"#define {nm} {v}"
        seen += 1
    assert seen > 40


def split_args(s):
    """Top-level comma split of a Rust call's argument text."""
    out, depth, cur = [], 0, ""
    for ch in s:
        if ch in "([{":
            depth += 1
        elif ch in ")]}":
            depth -= 1
        if ch == "," and depth == 0:
            out.append(cur)
            cur = ""
        else:
            cur += ch
    if cur.strip():
        out.append(cur)
    return out


def test_safe_layer_calls_declared_functions_with_their_arity():
    decl = rust_functions()
    calls = 0
    for path in sorted(SAFE.glob("*.rs")):
        text = re.sub(r"//[^\n]*", "", path.read_text())
        for m in re.finditer(r"sys::(rcu_[a-z0-9_]+)\s*\(", text):
            name = m.group(1)
            assert name in decl, f"{path.name}: sys::{name} is not declared"
            depth, i = 1, m.end()
            while depth:
                depth += {"(": 1, ")": -1}.get(text[i], 0)
                i += 1
            n = len(split_args(text[m.end():i - 1]))
            assert n == len(decl[name][1]), f"{path.name}: {name} takes {len(decl[name][1])} arguments, called with {n}"
            calls += 1
    assert calls >= 25
    used = set(re.findall(r"sys::(RCU_\w+)", "".join(p.read_text() for p in SAFE.glob("*.rs"))))
    consts = set(re.findall(r"pub const (RCU_\w+)", SYS.read_text()))
    assert used <= consts, sorted(used - consts)
