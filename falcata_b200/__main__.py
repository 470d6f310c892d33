"""``python -m falcata_b200`` - model-artifact utilities.

convert   rewrite a model between the LightGBM text format and the compressed binary FALB format (the
          input format is detected from the file's first bytes; both directions keep the model intact).

Parity: python-package/falcata/__main__.py (convert L14-47).
"""
from __future__ import annotations

import argparse
import sys
from pathlib import Path


def _cmd_convert(args: argparse.Namespace) -> int:
    import falcata_b200 as fb

    src, dst = Path(args.input), Path(args.output)
    booster = fb.Booster(model_file=str(src))
    fmt = args.format
    if fmt == "auto":
        suffixes = [x.lower() for x in dst.suffixes if x.lower() != ".gz"]
        fmt = "falb" if suffixes and suffixes[-1] == ".falb" else "txt"
    booster.save_model(str(dst), num_iteration=-1, format=fmt, f32_leaves=args.f32_leaves)
    a, b = src.stat().st_size, dst.stat().st_size
    print(f"{src} ({a} bytes) -> {dst} ({b} bytes, {fmt}), ratio {a / b if b else float('nan'):.2f}x")
    return 0


def main(argv: "list[str] | None" = None) -> int:
    ap = argparse.ArgumentParser(prog="falcata_b200")
    sub = ap.add_subparsers(dest="command", required=True)
    cv = sub.add_parser("convert", help="convert a model between txt and falb")
    cv.add_argument("input", help="model file to read (format detected from its content)")
    cv.add_argument("output", help="model file to write")
    cv.add_argument("--format", choices=("auto", "txt", "falb"), default="auto", help="output format; auto picks by the output extension")
    cv.add_argument("--f32-leaves", action="store_true", help="store leaf values as float32 (lossy, smaller)")
    cv.set_defaults(func=_cmd_convert)
    args = ap.parse_args(argv)
    return args.func(args)


if __name__ == "__main__":
    sys.exit(main())
