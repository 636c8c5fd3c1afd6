"""The C# glue under integration/ against the C header and the reference's Backend class (no .NET SDK exists here, so the
files cannot be compiled; these checks are textual).

  * NsB200Native.cs is what integration/gen_native_cs.py writes from include/ns_b200.h (not stale), imports every
    exported function exactly once, with the header's parameter count and integer widths;
  * NsB200Backend.cs overrides every abstract member of Backend (src/NeuralSharp/Backends/Backend.cs:66-282; the member list
    with parameter counts is the fixture tests/golden/backend_members.json) and every native call in it names an import
    and passes the right number of arguments.
"""
import json
import os
import re
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "integration"))
import gen_native_cs as gen  # noqa: E402

NATIVE = os.path.join(ROOT, "integration", "NsB200Native.cs")
BACKEND = os.path.join(ROOT, "integration", "NsB200Backend.cs")

WIDTH = {"int": {"int"}, "int32_t": {"int"}, "uint32_t": {"uint"}, "int64_t": {"long"}, "uint64_t": {"ulong"}, "float": {"float"}}


def _imports():
    text = open(NATIVE).read()
    found = re.findall(r"\[LibraryImport\(Library\)\]\s*public static partial (\w+) (\w+)\(([^)]*)\);", text)
    return {name: (ret, [p.strip() for p in params.split(",") if p.strip()]) for ret, name, params in found}, len(found)


def _split_args(s: str):
    args, depth, cur = [], 0, ""
    for ch in s:
        if ch in "([{":
            depth += 1
        elif ch in ")]}":
            depth -= 1
        if ch == "," and depth == 0:
            args.append(cur)
            cur = ""
        else:
            cur += ch
    if cur.strip():
        args.append(cur)
    return args


def test_native_file_is_current_and_complete():
    assert subprocess.run([sys.executable, os.path.join(ROOT, "integration", "gen_native_cs.py"), "--check"]).returncode == 0
    protos = gen.prototypes(open(os.path.join(ROOT, "include", "ns_b200.h")).read())
    imports, count = _imports()
    assert count == len(imports) == len(protos), "every export is imported exactly once"
    for ret, name, params in protos:
        cs_ret, cs_params = imports[name]
        assert cs_ret == ("nint" if ret == "const char*" else "int"), name
        assert len(cs_params) == len(params), f"{name}: {len(cs_params)} parameters in C#, {len(params)} in the header"
        for (ctype, _), cs in zip(params, cs_params):
            cs_type = cs.rsplit(" ", 1)[0]
            if ctype in WIDTH:
                assert cs_type in WIDTH[ctype], f"{name}: {ctype} bound as {cs_type}"
            elif ctype in gen.HANDLES:
                assert cs_type == "nint", f"{name}: handle bound as {cs_type}"
            else:
                assert ctype.endswith("*"), (name, ctype)
                elem = ctype.replace("const ", "")[:-1]
                if elem in WIDTH:
                    want = next(iter(WIDTH[elem]))
                    assert cs_type in (f"out {want}", f"{want}*"), f"{name}: {ctype} bound as {cs_type}"
                else:
                    assert cs_type in ("out nint", "void*", "byte*"), f"{name}: {ctype} bound as {cs_type}"


def test_backend_overrides_every_abstract_member_and_calls_real_imports():
    members = json.load(open(os.path.join(ROOT, "tests", "golden", "backend_members.json")))["members"]
    text = open(BACKEND).read()
    overrides = {}
    for name, params in re.findall(r"public override [\w<>\?\(\), \.]+?\s+(\w+)\s*\(([^)]*)\)", text, flags=re.S):
        overrides[name] = len([p for p in params.split(",") if p.strip()])
    for name in re.findall(r"public override \w+ (\w+)\s*=>", text):
        overrides.setdefault(name, None)
    for name, info in members.items():
        if info["kind"] == "abstract":
            assert name in overrides, f"Backend.{name} is abstract and not overridden"
        if name in overrides and info["parameters"] is not None:
            assert overrides[name] == info["parameters"], f"{name}: {overrides[name]} parameters, the reference has {info['parameters']}"
    for graph_member in ("SupportsGraphs", "BeginCapture", "EndCapture", "AbortCapture", "ReplayGraph", "DestroyGraph"):
        assert graph_member in overrides
    # every native call names an import and passes as many arguments as the import takes
    imports, _ = _imports()
    calls = 0
    for m in re.finditer(r"\b(ns_\w+)\(", text):
        name = m.group(1)
        if text[max(0, m.start() - 7):m.start()] == "nameof(":
            assert name in imports, f"nameof({name}) names no import"
            continue
        assert name in imports, f"{name} is called but not imported"
        depth, i = 1, m.end()
        while depth:
            depth += {"(": 1, ")": -1}.get(text[i], 0)
            i += 1
        args = _split_args(text[m.end():i - 1])
        assert len(args) == len(imports[name][1]), f"{name}: {len(args)} arguments passed, the import takes {len(imports[name][1])}"
        calls += 1
    assert calls >= 30
    # the operators of the decoder step go to the float32 surface, one entry point each
    for needed in ("ns_f32_batched_matmul", "ns_f32_scale_mask_softmax", "ns_f32_layernorm_fused", "ns_f32_bias_gelu", "ns_f32_decoder_mask",
                   "ns_f32_key_value_write", "ns_f32_gather", "ns_f32_argmax", "ns_f32_add_row_vector", "ns_f32_add", "ns_f32_affine",
                   "ns_f32_add_broadcast_scalar", "ns_f32_permute", "ns_f32_copy2d", "ns_f32_sample_rows", "ns_f32_penalize_rows",
                   "ns_f32_history_push", "ns_capture_begin", "ns_capture_end", "ns_capture_abort", "ns_graph_launch", "ns_graph_destroy"):
        assert re.search(rf"\b{needed}\(", text), f"{needed} is never called"
