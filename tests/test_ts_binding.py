"""The TypeScript glue is source only here (no JavaScript engine in the image), so what can be held to the library is:
every koffi prototype string of ``mlfw_b200/ts/binding.ts`` against the declarations of ``include/b200q.h`` (same
functions, same argument counts, same scalar types in the same positions), every binding name the other ``.ts`` files
call against the names binding.ts defines, and the registration calls ``register.ts`` makes against the reference's
registry signatures (names only)."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TS = os.path.join(ROOT, "mlfw_b200", "ts")
SCALARS = {"int", "int64_t", "double", "float", "size_t", "uint64_t"}


def header_prototypes():
    text = re.sub(r"/\*.*?\*/", "", open(os.path.join(ROOT, "include", "b200q.h")).read(), flags=re.S)
    out = {}
    for ret, name, args in re.findall(r"^\s*([A-Za-z_][\w\s\*]*?)\b(b200q_\w+)\s*\(([^;{]*?)\)\s*;", text, flags=re.M):
        kinds = []
        for a in [x.strip() for x in args.split(",")] if args.strip() and args.strip() != "void" else []:
            ty = " ".join(a.split()).rsplit(" ", 1)[0] if not a.endswith("*") else a
            ty = re.sub(r"\b\w+$", "", a).strip() if "*" not in a.split()[-1] else a
            kinds.append("ptr" if "*" in a else ty.replace("const", "").strip())
        ret = " ".join(ret.split())
        out[name] = ("ptr" if "*" in ret else ret, kinds)
    return out


def binding_prototypes():
    text = open(os.path.join(TS, "binding.ts")).read()
    out, keys = {}, {}
    for key, proto in re.findall(r"^\s*(\w+): f\('([^']+)'\),", text, flags=re.M):
        m = re.match(r"(.*?)\b(b200q_\w+)\((.*)\)$", proto)
        ret, name, args = m.group(1).strip(), m.group(2), m.group(3)
        kinds = []
        for a in [x.strip() for x in args.split(",")] if args.strip() else []:
            a = a.replace("_Out_", "").strip()
            kinds.append("ptr" if "*" in a else a.rsplit(" ", 1)[0].replace("const", "").strip())
        out[name] = ("ptr" if ("*" in ret or ret == "str") else ret, kinds)
        keys[key] = name
    return out, keys


def test_binding_ts_matches_the_header():
    hdr = header_prototypes()
    ts, keys = binding_prototypes()
    assert len(hdr) >= 70
    assert set(ts) == set(hdr), f"only in header: {sorted(set(hdr) - set(ts))}; only in binding.ts: {sorted(set(ts) - set(hdr))}"
    for name, (ret, kinds) in hdr.items():
        tret, tkinds = ts[name]
        assert tret == ret, f"{name}: returns {ret} in the header, {tret} in binding.ts"
        assert tkinds == kinds, f"{name}: arguments {kinds} in the header, {tkinds} in binding.ts"
        assert all(k == "ptr" or k in SCALARS for k in kinds), (name, kinds)
    assert len(set(keys)) == len(keys) == len(hdr)


def test_every_binding_name_used_by_the_glue_exists():
    _, keys = binding_prototypes()
    for fname in ("plan.ts", "runtime_module.ts", "register.ts"):
        text = open(os.path.join(TS, fname)).read()
        used = set(re.findall(r"\b(?:bind|b|s\.b|this\.b)\.([a-zA-Z0-9]+)\(", text))
        missing = {u for u in used if u not in keys}
        assert not missing, f"{fname} calls binding entries that binding.ts does not define: {sorted(missing)}"


def test_register_ts_uses_the_reference_registries():
    text = open(os.path.join(TS, "register.ts")).read()
    assert "registerBackend(B200_KIND" in text and "DispatchKey.CUSTOM_1" in text and "new Library('mlc', 'IMPL')" in text
    for op in ("b200_quantize_per_token", "b200_dequantize_per_token", "b200_int8_linear"):
        assert text.count(op) >= 2           # a schema and an implementation
    for member in ("instantiate", "runSync", "runAsync", "isAsync"):
        assert re.search(rf"\b{member}\(", text)
    plan = open(os.path.join(TS, "plan.ts")).read()
    assert "export function planFromProgram" in plan and "export function programOf" in plan
