"""Puts the reference's own Lazy Attention module where the same-box comparator looks for it.

    python oracle/make_ref.py <path to the reference checkout>

Copies ``lazy_attention_triton.py`` (the one implementation file of the reference's checkout) unmodified
into ``oracle/_ref/``.  That folder is listed in ``.gitignore``: the file never enters this repository's
history, it only has to be present on the machine that runs ``python bench.py --lazy-compare``, where the
reference's Triton kernels are JIT-compiled for the local GPU and timed beside this library's.
TEST / MEASUREMENT INFRASTRUCTURE ONLY: nothing in the shipped package imports it.
"""
import os
import shutil
import sys


def main() -> None:
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    src = os.path.join(sys.argv[1], "lazy_attention_triton.py")
    if not os.path.exists(src):
        sys.exit(f"{src} not found")
    dst_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")
    os.makedirs(dst_dir, exist_ok=True)
    shutil.copyfile(src, os.path.join(dst_dir, "lazy_attention_triton.py"))
    print("copied", src, "->", dst_dir)


if __name__ == "__main__":
    main()
