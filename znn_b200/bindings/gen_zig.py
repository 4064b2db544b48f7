"""Regenerates the `pub extern fn` block of cuda.zig from include/znn_cuda.h (the hand-written head of the file, up to
the first `pub extern fn`, is kept).  Run after the header changed:  python znn_b200/bindings/gen_zig.py
tests/test_cabi_symbols.py checks that the two stay in step."""
import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))
HEADER = os.path.join(HERE, "..", "..", "include", "znn_cuda.h")
ZIG = os.path.join(HERE, "cuda.zig")

SCALAR = {"int": "c_int", "float": "f32", "double": "f64", "size_t": "usize", "long long": "c_longlong",
          "unsigned long long": "c_ulonglong", "unsigned": "c_uint", "unsigned int": "c_uint", "int32_t": "i32",
          "int64_t": "i64", "uint8_t": "u8", "uint32_t": "u32", "char": "u8"}
OUT_SCALARS = {"count", "status", "used", "high_water", "capacity", "total_floats", "offset", "generation", "n",
               "kernel_ms", "launches", "flops", "num_images", "rows_out", "cols_out", "num_labels", "loss_out", "world", "rank"}


def zig_type(ctype, name):
    ctype = ctype.strip()
    const = ctype.startswith("const ")
    if const:
        ctype = ctype[6:].strip()
    stars = ctype.count("*")
    base = ctype.replace("*", "").strip()
    if stars == 0:
        return SCALAR[base]
    if base == "void":
        inner = "?*const anyopaque" if const else "?*anyopaque"
        return inner if stars == 1 else "*" + ("?*anyopaque")
    if base.startswith("znn_"):
        return ("?*" + base) if stars == 1 else ("*?*" + base)
    z = SCALAR[base]
    if stars == 2:
        return "*?[*]" + z
    if base == "char":
        return "[*:0]const u8" if const else "[*]u8"
    if name in OUT_SCALARS and not const:
        return "?*" + z
    return ("?[*]const " if const else "?[*]") + z


def declarations(text):
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    text = re.sub(r"^\s*#.*$", " ", text, flags=re.M)
    for m in re.finditer(r"\bint\s+(znn_\w+)\s*\(([^)]*)\)\s*;", text):
        name, args = m.group(1), " ".join(m.group(2).split())
        params = []
        if args and args != "void":
            for a in args.split(","):
                a = a.strip()
                pm = re.match(r"(.*?)(\w+)$", a)
                params.append((pm.group(1).strip(), pm.group(2)))
        yield name, params


def main():
    head = open(ZIG).read()
    head = head[:head.index("pub extern fn")]
    lines = []
    for name, params in declarations(open(HEADER).read()):
        ps = ", ".join(f"{pn}: {zig_type(pt, pn)}" for pt, pn in params)
        lines.append(f"pub extern fn {name}({ps}) c_int;")
    open(ZIG, "w").write(head + "\n".join(lines) + "\n")
    print(f"{len(lines)} declarations written to {ZIG}")


if __name__ == "__main__":
    main()
