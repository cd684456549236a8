#!/usr/bin/env python
"""Copy the reference's efficiency kernels (five small Triton files and the op wrappers) from a
WSVD checkout into baseline/_ref/, unmodified, so that `bench.py --triton-reference` can time them
on the GPU box beside this library.  baseline/_ref/ is git-ignored: the reference's source never
enters this repository's history.

    python baseline/fetch_ref.py [path to the WSVD checkout]
"""
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEFAULT_SRC = os.environ.get("WSVD_REFERENCE", "/root/reference")
FILES = [
    "efficiency/kernel/flash_decoding.py",
    "efficiency/kernel/flash_decoding_stage1.py",
    "efficiency/kernel/flash_decoding_stage2.py",
    "efficiency/kernel/flash_int8_latent_per_head_decoding_rope_stage1.py",
    "efficiency/kernel/flash_latent_per_head_decoding_rope_stage1.py",
    "efficiency/kernel/flash_latent_per_head_decoding_stage2.py",
]


def main(src: str = DEFAULT_SRC) -> int:
    if not os.path.isdir(src):
        print(f"no WSVD checkout at {src}: nothing copied")
        return 1
    for rel in FILES:
        dst = os.path.join(HERE, "_ref", rel)
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        shutil.copyfile(os.path.join(src, rel), dst)
    init = os.path.join(HERE, "_ref", "efficiency", "kernel", "__init__.py")
    if os.path.exists(os.path.join(src, "efficiency/kernel/__init__.py")):
        shutil.copyfile(os.path.join(src, "efficiency/kernel/__init__.py"), init)
    print(f"copied {len(FILES)} files into {os.path.join(HERE, '_ref')}")
    return 0


if __name__ == "__main__":
    sys.exit(main(*sys.argv[1:2]))
