"""CPU test of the Common Lisp backend file (`lisp/b200.lisp`) against the C header: every
`foreign-funcall` in it must name a function `include/caten_b200.h` declares, with the same number of
arguments, CFFI types that match the C types, and the right return type; the two `defcstruct`s must
list the header's struct fields in order.  (The file itself cannot be run here: there is no Common
Lisp implementation on the build machine; this keeps it honest about the ABI.)"""
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "caten_b200.h")
LISP = os.path.join(ROOT, "lisp", "b200.lisp")


def strip_c_comments(src):
    src = re.sub(r"/\*.*?\*/", " ", src, flags=re.S)
    return "\n".join(line for line in src.splitlines() if not line.lstrip().startswith("#"))


def c_type_to_cffi(ctype):
    t = " ".join(ctype.replace("const", " ").split())
    if "*" in t:
        return {":pointer"} | ({":string"} if t.replace(" ", "") == "char*" else set())
    return {"int": {":int"}, "unsigned": {":uint", ":unsigned-int"}, "int64_t": {":int64"}, "size_t": {":size"},
            "float": {":float"}, "double": {":double"}, "int32_t": {":int32"}, "uint32_t": {":uint32"}}[t]


def header_functions():
    src = strip_c_comments(open(HEADER).read())
    src = re.sub(r"typedef struct \{.*?\} \w+;", " ", src, flags=re.S)
    out = {}
    for m in re.finditer(r"([A-Za-z_][\w\s\*]*?)\b(caten_b200_\w+)\s*\(([^;{]*?)\)\s*;", src):
        ret, name, args = m.group(1).strip(), m.group(2), m.group(3).strip()
        params = []
        if args and args != "void":
            for a in args.split(","):
                a = a.strip()
                a = re.sub(r"\b\w+$", "", a).strip() if not a.endswith("*") else a   # drop the parameter name
                params.append(a)
        out[name] = (ret, params)
    return out


def lisp_without_comments_and_docstrings(src):
    src = re.sub(r"#\|.*?\|#", " ", src, flags=re.S)
    return "\n".join(line.split(";")[0] if '"' not in line.split(";")[0] or line.split(";")[0].count('"') % 2 == 0 else line
                     for line in src.splitlines())


def sexp_end(src, start):
    depth, i, in_str = 0, start, False
    while i < len(src):
        c = src[i]
        if in_str:
            if c == "\\":
                i += 1
            elif c == '"':
                in_str = False
        elif c == '"':
            in_str = True
        elif c == "(":
            depth += 1
        elif c == ")":
            depth -= 1
            if depth == 0:
                return i + 1
        i += 1
    raise AssertionError("unbalanced s-expression")


def top_level_items(body):
    """Splits the inside of a list into its top-level items."""
    items, i = [], 0
    while i < len(body):
        c = body[i]
        if c.isspace():
            i += 1
        elif c == "(":
            j = sexp_end(body, i)
            items.append(body[i:j]); i = j
        elif c == '"':
            j = i + 1
            while body[j] != '"':
                j += 2 if body[j] == "\\" else 1
            items.append(body[i:j + 1]); i = j + 1
        else:
            j = i
            while j < len(body) and not body[j].isspace() and body[j] not in "()":
                j += 1
            if body[i:j] in ("'", "`", ",", "#'"):
                k = sexp_end(body, j) if body[j] == "(" else j
                items.append(body[i:k]); i = k
            else:
                items.append(body[i:j]); i = j
    return items


def lisp_calls():
    src = lisp_without_comments_and_docstrings(open(LISP).read())
    calls = []
    for m in re.finditer(r"\(foreign-funcall\s", src):
        end = sexp_end(src, m.start())
        items = top_level_items(src[m.start() + 1:end - 1])[1:]
        name = items[0].strip('"')
        rest = items[1:]
        assert len(rest) % 2 == 1, f"{name}: expected type/value pairs and a return type, got {rest}"
        types = [rest[i] for i in range(0, len(rest) - 1, 2)]
        calls.append((name, types, rest[-1], src.count("\n", 0, m.start()) + 1))
    return calls


def test_every_foreign_funcall_matches_the_header():
    decl = header_functions()
    calls = lisp_calls()
    assert len(calls) >= 30
    for name, types, ret, line in calls:
        assert name in decl, f"b200.lisp:{line}: {name} is not declared in caten_b200.h"
        cret, cparams = decl[name]
        assert len(types) == len(cparams), f"b200.lisp:{line}: {name} takes {len(cparams)} arguments, called with {len(types)}"
        for k, (lt, ct) in enumerate(zip(types, cparams)):
            assert lt in c_type_to_cffi(ct), f"b200.lisp:{line}: {name} argument {k}: {lt} against C type '{ct}'"
        assert ret in c_type_to_cffi(cret), f"b200.lisp:{line}: {name} returns '{cret}', bound as {ret}"


def test_the_backend_uses_the_entry_points_of_the_path():
    used = {c[0] for c in lisp_calls()}
    for needed in ("caten_b200_init", "caten_b200_last_error", "caten_b200_malloc", "caten_b200_free", "caten_b200_h2d",
                   "caten_b200_d2h", "caten_b200_d2d", "caten_b200_weight_upload", "caten_b200_weight_upload_device",
                   "caten_b200_weight_dequant", "caten_b200_linear", "caten_b200_layernorm", "caten_b200_embed",
                   "caten_b200_attention_ex", "caten_b200_argmax", "caten_b200_relu_matmul", "caten_b200_eval_expr",
                   "caten_b200_gpt2_create", "caten_b200_gpt2_step", "caten_b200_gpt2_destroy", "caten_b200_dist_init",
                   "caten_b200_dist_bcast_weights", "caten_b200_dist_gather_ids", "caten_b200_dist_shard"):
        assert needed in used, needed


def header_struct_fields(name):
    src = strip_c_comments(open(HEADER).read())
    body = re.search(r"typedef struct \{([^}]*)\} " + name + ";", src).group(1)
    fields = []
    for stmt in body.split(";"):
        stmt = stmt.strip()
        if not stmt:
            continue
        # "const float *const *ln1_g, *const *ln1_b" or "int32_t n_layers, d_model" or "int64_t shape[6]"
        first, *more = stmt.split(",")
        pat = r"(\w+)\s*(\[[^\]]*\]\s*)*$"
        names = [re.search(pat, first).group(1)] + [re.search(pat, x).group(1) for x in more]
        fields += names
    return fields


@pytest.mark.parametrize("cname,lname", [("caten_b200_gpt2_desc", "caten-b200-gpt2-desc"), ("caten_b200_expr", "caten-b200-expr")])
def test_defcstruct_fields_follow_the_header(cname, lname):
    src = lisp_without_comments_and_docstrings(open(LISP).read())
    m = re.search(r"\(defcstruct " + lname + r"\s", src)
    items = top_level_items(src[m.start() + 1:sexp_end(src, m.start()) - 1])[2:]
    lisp_fields = [top_level_items(it[1:-1])[0].replace("-", "_") for it in items]
    assert lisp_fields == header_struct_fields(cname)


def test_registration_forms_are_present():
    src = open(LISP).read()
    assert "(define-backend :b200 B200Buffer B200Runtime B200-Renderer B200-Auto-Scheduler t)" in src
    for generic in ("open-buffer", "close-buffer", "transfer-from-array", "transfer-into-array", "copy-buffer-value", "bref",
                    "%render-kernel", "%compile-kernel", "runtime-invoke-jit-kernel", "realize-node"):
        assert re.search(r"\(defmethod " + re.escape(generic) + r"[\s(]", src), generic
