"""Writes tests/golden/backend_members.json: the abstract and virtual members of the reference's Backend class
(src/NeuralSharp/Backends/Backend.cs:66-282) with their parameter counts, read from the reference checkout.

    python tests/golden/make_backend_members.py /path/to/reference

tests/test_integration_cs.py holds the C# backend of integration/ to this list (every abstract member overridden with
the same number of parameters), so the check runs where the reference is not available.
"""
import json
import os
import re
import sys


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_backend_members.py <checkout of the reference>")
    root = sys.argv[1]
    text = open(os.path.join(root, "src", "NeuralSharp", "Backends", "Backend.cs")).read()
    body = text[text.index("internal abstract class Backend"):text.index("internal static class CounterRandom")]
    members = {}
    for kind, name, params in re.findall(r"public\s+(abstract|virtual)\s+[\w<>\?\(\), \.]+?\s+(\w+)\s*\(([^)]*)\)", body, flags=re.S):
        count = 0 if not params.strip() else len([p for p in params.split(",") if p.strip()])
        members[name] = {"kind": kind, "parameters": count}
    for kind, name in re.findall(r"public\s+(abstract|virtual)\s+[\w<>\?]+\s+(\w+)\s*=>", body):
        members.setdefault(name, {"kind": kind, "parameters": None})
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "backend_members.json")
    json.dump({"source": "src/NeuralSharp/Backends/Backend.cs", "members": members}, open(out, "w"), indent=1, sort_keys=True)
    print(f"{len(members)} members -> {out}")


if __name__ == "__main__":
    main()
