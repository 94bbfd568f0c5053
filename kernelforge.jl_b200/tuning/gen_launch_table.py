"""Generates csrc/launch_table.h from tuning/launch_table.json.

    python kernelforge.jl_b200/tuning/gen_launch_table.py

The JSON is the committed, human-editable launch table (the counterpart of the reference's
data/tuning/<Arch>_inline.jl artifacts); the header is what the library compiles in.
"""
import json
import os

HERE = os.path.dirname(os.path.abspath(__file__))
U64_MAX = "18446744073709551615ull"


def main():
    with open(os.path.join(HERE, "launch_table.json")) as fh:
        table = json.load(fh)
    prim = table["primitives"]
    rows = table["rows"]
    lines = [
        "// B200 launch table: (primitive, element bytes, input size) -> (threads, items, CTAs per SM).",
        "// GENERATED from tuning/launch_table.json by tuning/gen_launch_table.py; edit the JSON, not this file.",
        "// The first row that matches the primitive and element size and whose bound covers the input wins;",
        "// elem_bytes 0 matches any element size (key + payload bytes for sorts).",
        "#pragma once",
        "#include <stdint.h>",
        "",
        "namespace kf {",
        "struct LaunchRow {",
        "    int primitive;       // kf_primitive",
        "    int elem_bytes;      // 0 = any",
        "    uint64_t max_bytes;  // row applies to inputs of at most this many bytes",
        "    int threads, items, blocks_per_sm;",
        "};",
        "static const LaunchRow kLaunchTable[] = {",
    ]
    for r in rows:
        mb = U64_MAX if r["max_bytes"] is None else "%dull" % r["max_bytes"]
        lines.append("    {%d, %d, %s, %d, %d, %d}," % (prim[r["primitive"]], r["elem_bytes"], mb, r["threads"], r["items"],
                                                       r["blocks_per_sm"]))
    lines += ["};", "static const int kNumLaunchRows = %d;" % len(rows), "}  // namespace kf", ""]
    out = os.path.join(HERE, "..", "csrc", "launch_table.h")
    with open(out, "w") as fh:
        fh.write("\n".join(lines))
    print("wrote", os.path.normpath(out), "with", len(rows), "rows")


if __name__ == "__main__":
    main()
