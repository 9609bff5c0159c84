"""The Rust side of the boundary, kept as source: oxidizr_b200/rust/oxz-dpstep-sys/src/lib.rs declares every entry
point and every struct of include/oxz_dpstep.h for the reference's own language. No Rust toolchain is needed to check
it: both files are parsed here and compared - every function present with the same argument count and types, every
struct with the same fields in the same order, every status / enum constant with the same value."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "oxz_dpstep.h")
CRATE = os.path.join(ROOT, "oxidizr_b200", "rust", "oxz-dpstep-sys")

SCALARS = {"int32_t": "i32", "uint32_t": "u32", "int64_t": "i64", "uint64_t": "u64", "uint8_t": "u8", "double": "f64",
           "float": "f32", "char": "c_char", "void": "c_void", "size_t": "usize"}


def strip_comments(text: str) -> str:
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    return re.sub(r"//[^\n]*", " ", text)


def c_type_to_rust(ctype: str, array: bool = False) -> str:
    """One C parameter or field type (name removed) as the Rust FFI type this crate must use."""
    t = " ".join(ctype.replace("*", " * ").split())
    fn = {"oxz_rank_body": "oxz_rank_body"}
    if t in fn:
        return fn[t]
    toks = t.split()
    # read right to left: pointers wrap what stands to their left
    base_const = False
    base = None
    out = None
    i = 0
    # base type: optional const, name, optional const
    if toks[i] == "const":
        base_const = True
        i += 1
    base = toks[i]
    i += 1
    if i < len(toks) and toks[i] == "const":
        base_const = True
        i += 1
    out = SCALARS.get(base, base)
    const_here = base_const
    while i < len(toks):
        assert toks[i] == "*", (ctype, toks)
        i += 1
        out = ("*const " if const_here else "*mut ") + out
        const_here = False
        if i < len(toks) and toks[i] == "const":
            const_here = True
            i += 1
    if array:  # a C array parameter is a pointer to its element
        out = ("*const " if const_here or base_const else "*mut ") + out
    return out


def split_params(arglist: str):
    arglist = arglist.strip()
    if arglist in ("", "void"):
        return []
    out = []
    for part in arglist.split(","):
        part = part.strip()
        m = re.match(r"^(.*?)([A-Za-z_][A-Za-z0-9_]*)\s*(\[\s*\d*\s*\])?$", part)
        assert m, part
        ctype, name, arr = m.group(1).strip(), m.group(2), m.group(3)
        out.append((name, c_type_to_rust(ctype, array=arr is not None)))
    return out


def parse_header():
    text = strip_comments(open(HEADER).read())
    text = re.sub(r"#[^\n]*", " ", text)
    structs, functions, constants = {}, {}, {}
    for m in re.finditer(r"typedef\s+struct\s+(\w+)\s*\{(.*?)\}\s*(\w+)\s*;", text, flags=re.S):
        fields = []
        for decl in m.group(2).split(";"):
            decl = decl.strip()
            if not decl:
                continue
            # "double a, b;" declares several fields of one type
            first = re.match(r"^(.*?)([A-Za-z_]\w*)\s*(\[\s*(\d+)\s*\])?$", decl.split(",")[0].strip())
            ctype = first.group(1).strip()
            for k, piece in enumerate(decl.split(",")):
                piece = piece.strip()
                if k == 0:
                    name, n, stars = first.group(2), first.group(4), 0
                else:  # a later declarator of the same declaration: "*name" or "name[n]"
                    mm = re.match(r"^(\**)\s*([A-Za-z_]\w*)\s*(\[\s*(\d+)\s*\])?$", piece)
                    name, n, stars = mm.group(2), mm.group(4), len(mm.group(1))
                rt = c_type_to_rust(ctype + " *" * stars)
                fields.append((name, f"[{rt}; {n}]" if n else rt))
        structs[m.group(3)] = fields
    for m in re.finditer(r"typedef\s+enum\s+\w+\s*\{(.*?)\}\s*\w+\s*;", text, flags=re.S):
        nxt = 0
        for item in m.group(1).split(","):
            item = item.strip()
            if not item:
                continue
            if "=" in item:
                name, val = [x.strip() for x in item.split("=")]
                nxt = int(val, 0)
            else:
                name = item
            constants[name] = nxt
            nxt += 1
    for m in re.finditer(r"#define\s+(OXZ_[A-Z0-9_]+)\s+(\d+)u?\b", strip_comments(open(HEADER).read())):
        constants[m.group(1)] = int(m.group(2))
    body = re.sub(r"typedef\s+(struct|enum)\s+\w+\s*\{.*?\}\s*\w+\s*;", " ", text, flags=re.S)
    body = re.sub(r"typedef[^;]*;", " ", body)
    for m in re.finditer(r"([A-Za-z_][\w\s\*]*?)\b(oxz_[a-z0-9_]+)\s*\(([^)]*)\)\s*;", body):
        ret = " ".join(m.group(1).split())
        functions[m.group(2)] = (split_params(m.group(3)), "()" if ret == "void" else c_type_to_rust(ret))
    return structs, functions, constants


def parse_rust():
    text = open(os.path.join(CRATE, "src", "lib.rs")).read()
    text = re.sub(r"//[^\n]*", " ", text)
    structs, functions, constants = {}, {}, {}
    for m in re.finditer(r"#\[repr\(C\)\]\s*(?:#\[derive\([^)]*\)\]\s*)?pub\s+struct\s+(\w+)\s*\{(.*?)\}", text, flags=re.S):
        fields = []
        for f in m.group(2).split(","):
            f = f.strip()
            if not f:
                continue
            name, ty = f.replace("pub ", "", 1).split(":", 1)
            fields.append((name.strip(), " ".join(ty.split())))
        structs[m.group(1)] = fields
    for m in re.finditer(r"pub\s+const\s+(OXZ_[A-Z0-9_]+)\s*:\s*\w+\s*=\s*(\d+)\s*;", text):
        constants[m.group(1)] = int(m.group(2))
    ext = re.search(r'extern\s+"C"\s*\{(.*)\}', text, flags=re.S).group(1)
    for m in re.finditer(r"pub\s+fn\s+(oxz_[a-z0-9_]+)\s*\((.*?)\)\s*(?:->\s*([^;]+?))?\s*;", ext, flags=re.S):
        params = []
        for prm in [x.strip() for x in m.group(2).split(",") if x.strip()]:
            name, ty = prm.split(":", 1)
            params.append((name.strip(), " ".join(ty.split())))
        functions[m.group(1)] = (params, " ".join((m.group(3) or "()").split()))
    return structs, functions, constants


def test_every_entry_point_is_declared_with_the_same_arguments():
    _, hf, _ = parse_header()
    _, rf, _ = parse_rust()
    assert len(hf) >= 90
    missing = sorted(set(hf) - set(rf))
    extra = sorted(set(rf) - set(hf))
    assert not missing, f"declared in the header but not in lib.rs: {missing}"
    assert not extra, f"in lib.rs but not in the header: {extra}"
    for name, (params, ret) in hf.items():
        rparams, rret = rf[name]
        assert len(params) == len(rparams), f"{name}: {len(params)} arguments in the header, {len(rparams)} in lib.rs"
        assert [t for _, t in params] == [t for _, t in rparams], f"{name}: {params} vs {rparams}"
        assert ret == rret, f"{name}: returns {ret} in the header, {rret} in lib.rs"


def test_every_struct_has_the_same_fields_in_the_same_order():
    hs, _, _ = parse_header()
    rs, _, _ = parse_rust()
    assert len(hs) >= 15
    for name, fields in hs.items():
        assert name in rs, f"struct {name} is missing from lib.rs"
        assert fields == rs[name], f"{name}: header {fields} vs lib.rs {rs[name]}"
    for opaque in ("oxz_comm", "oxz_plan", "oxz_loader"):
        assert opaque in rs and rs[opaque] == [("_private", "[u8; 0]")], opaque


def test_every_constant_has_the_same_value():
    _, _, hc = parse_header()
    _, _, rc = parse_rust()
    assert len(hc) >= 30
    for name, value in hc.items():
        assert rc.get(name) == value, f"{name}: {value} in the header, {rc.get(name)} in lib.rs"


def test_the_safe_wrapper_calls_only_declared_entry_points():
    _, hf, _ = parse_header()
    text = open(os.path.join(CRATE, "src", "safe.rs")).read()
    used = set(re.findall(r"\bsys::(oxz_[a-z0-9_]+)\s*\(", text))
    assert len(used) >= 20
    assert not used - set(hf), sorted(used - set(hf))
    # the calls LitTrainer's step makes (src/trainer.rs:184-193, 254, 520-527, 573-587, 649, 666-681)
    for needed in ("oxz_plan_create", "oxz_state_alloc", "oxz_grads_flatten_async", "oxz_step", "oxz_scaler_record_step",
                   "oxz_lr_at", "oxz_spike_judge", "oxz_decay_excludes", "oxz_comm_abort", "oxz_grad_norms_per_tensor"):
        assert needed in used, needed
