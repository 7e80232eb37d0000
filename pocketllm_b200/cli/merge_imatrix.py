"""`python -m pocketllm_b200.cli.merge_imatrix OUT IN1 IN2 ...`: sum importance matrices."""
from __future__ import annotations

import sys

from ..formats import imatrix


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    if len(argv) < 2:
        print("usage: merge_imatrix OUT IN [IN ...]", file=sys.stderr)
        return 2
    acc = imatrix.merge(argv[1:], argv[0])
    print(f"merged {len(argv) - 1} files, {len(acc.sum2)} tensors -> {argv[0]}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
