"""Write a small synthetic click-through data set in the native text format (``label; group key ...;``),
in place of the data sets that the reference's tutorial downloads:

    python examples/linear/make_data.py                                        # data/ctr/{train,test}/part-NN
    python examples/linear/make_data.py --format libsvm --out data/rcv1        # index:value pairs (rcv1 example)
    python examples/linear/make_data.py --format criteo --out data/criteo      # click-log lines (criteo example)

Ids follow a Zipf-like law, labels come from a sparse ground-truth model with logistic noise."""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from parameter_server_b200.utils.textdata import write_criteo, write_libsvm, write_sparse_binary  # noqa: E402


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--format", default="sparse_binary", choices=["sparse_binary", "libsvm", "criteo"])
    ap.add_argument("--out", default="data/ctr")
    ap.add_argument("--files", type=int, default=4)
    ap.add_argument("--rows", type=int, default=5000, help="rows per file")
    ap.add_argument("--nnz", type=int, default=24, help="nonzeros per row")
    ap.add_argument("--features", type=int, default=20000)
    args = ap.parse_args(argv)
    tr, te = os.path.join(args.out, "train"), os.path.join(args.out, "test")
    if args.format == "criteo":
        train, test = write_criteo(tr, args.files, args.rows, seed=1), write_criteo(te, 1, args.rows, seed=2)
    else:
        write = write_libsvm if args.format == "libsvm" else write_sparse_binary
        train, _ = write(tr, args.files, args.rows, args.nnz, args.features, seed=1)
        test, _ = write(te, 1, args.rows, args.nnz, args.features, seed=1)
    print("wrote", len(train), "training files and", len(test), "test file under", args.out)


if __name__ == "__main__":
    main()
