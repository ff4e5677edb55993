"""Write a small synthetic click-through data set in the native text format (``label; group key ...;``),
in place of the data sets that the reference's tutorial downloads:

    python examples/linear/make_data.py            # data/ctr/train/part-00.. and data/ctr/test/part-00..

Ids follow a Zipf-like law, labels come from a sparse ground-truth model with logistic noise."""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from parameter_server_b200.utils.textdata import write_sparse_binary  # noqa: E402


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--out", default="data/ctr")
    ap.add_argument("--files", type=int, default=4)
    ap.add_argument("--rows", type=int, default=5000, help="rows per file")
    ap.add_argument("--nnz", type=int, default=24, help="nonzeros per row")
    ap.add_argument("--features", type=int, default=20000)
    args = ap.parse_args(argv)
    train, _ = write_sparse_binary(os.path.join(args.out, "train"), args.files, args.rows, args.nnz, args.features, seed=1)
    test, _ = write_sparse_binary(os.path.join(args.out, "test"), 1, args.rows, args.nnz, args.features, seed=1)
    print("wrote", len(train), "training files and", len(test), "test file under", args.out)


if __name__ == "__main__":
    main()
