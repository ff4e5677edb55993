"""Two small data tools, with the reference's flag names (``-input -output -format``):

* ``show``     print the first examples of a text file as parsed (slots, keys, values): the debugging printer
               ``data/show_example.h:8-18``;
* ``convert``  text files -> one record file of serialised examples plus ``<output>.info`` with the per-slot
               statistics (what ``data/text2proto.h:4-39`` sketches): ``<output>.recordio`` can then be named in a
               configuration with ``format: PROTO``. ``-to bin`` writes a binary matrix instead
               (``<output>.index .offset .label [.value] .info``, 64-bit ids): name ``<output>`` with ``format: BIN``
               and the GPU application maps it and reads minibatches without parsing.

    python -m parameter_server_b200.utils.datatool show -input part-0 -format libsvm -n 3
    python -m parameter_server_b200.utils.datatool convert -input 'data/part-.*' -output data/all -format criteo
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def _args(argv):
    ap = argparse.ArgumentParser(prog="datatool", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("cmd", choices=["show", "convert"])
    ap.add_argument("-input", "--input", required=True, help="file name (show) or file pattern (convert); stdin for show")
    ap.add_argument("-output", "--output", default="", help="convert: prefix of the files written")
    ap.add_argument("-format", "--format", default="libsvm",
                    help="libsvm, adfea, terafea, criteo, vw, dense, sparse, sparse_binary")
    ap.add_argument("-n", "--n", type=int, default=3, help="show: how many examples")
    ap.add_argument("-to", "--to", default="recordio", choices=["recordio", "bin"],
                    help="convert: record file of examples, or a binary matrix (format: BIN, read without parsing)")
    return ap.parse_args(argv)


def show(args, out=None) -> int:
    out = out or sys.stdout
    from ..system import core
    fmt = args.format.upper()
    lines = sys.stdin if args.input == "stdin" else open(args.input)
    shown = 0
    for line in lines:
        ex = core.parse_example(line.rstrip("\n"), fmt)
        if ex is None:
            continue
        print(json.dumps(ex, default=lambda a: a.tolist() if hasattr(a, "tolist") else str(a)), file=out)
        shown += 1
        if shown >= args.n:
            break
    return shown


def convert(args, out=None) -> int:
    out = out or sys.stdout
    from ..system import core
    if not args.output:
        raise SystemExit("convert needs -output")
    fmt = args.format.upper()
    files = list(core.search_files([args.input]))
    if os.path.dirname(args.output):
        os.makedirs(os.path.dirname(args.output), exist_ok=True)
    if args.to == "bin":
        from .binfmt import BinWriter
        w = BinWriter(args.output)
        reader = core.StreamReader(files, "TEXT", fmt, True)
        while True:
            got = reader.read_matrices(65536)
            if got is None:
                break
            if len(got[0]) and got[1]:
                w.add(got)
        w.close()
        print(f"{w.rows} examples, {w.nnz} nonzeros from {len(files)} file(s) -> {args.output}.{{index,offset,label,info}}", file=out)
        return w.rows
    n = core.text_to_records(files, fmt, args.output + ".recordio")
    info = core.SlotReader(files, fmt, "").read()
    with open(args.output + ".info", "w") as f:
        json.dump(info, f, indent=1)
    print(f"{n} examples from {len(files)} file(s) -> {args.output}.recordio, {args.output}.info", file=out)
    return n


def main(argv=None) -> int:
    args = _args(sys.argv[1:] if argv is None else argv)
    (show if args.cmd == "show" else convert)(args)
    return 0


if __name__ == "__main__":
    sys.exit(main())
