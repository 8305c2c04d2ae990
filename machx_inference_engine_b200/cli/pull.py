"""``ie pull NAME``: resolve a model name to a local GGUF path.

The reference shells out to a download script (scripts/ie-pull, src/cli/main.cpp:118-131).  This build runs on
machines without network access, so ``pull`` only resolves names against the local model directory (exact file,
NAME.gguf, first shard of a split set, or a directory holding one of those) and explains where to put the file
otherwise; it never opens a network connection.
"""
from __future__ import annotations

import glob
import os
import sys


def resolve(name: str, model_dir: str):
    cands = [name, os.path.join(model_dir, name), os.path.join(model_dir, name + ".gguf")]
    for c in cands:
        if os.path.isfile(c):
            return c
        if os.path.isdir(c):
            files = sorted(glob.glob(os.path.join(c, "*.gguf")))
            first = [f for f in files if "-00001-of-" in f] or files
            if first:
                return first[0]
    shards = sorted(glob.glob(os.path.join(model_dir, name + "-00001-of-*.gguf")))
    return shards[0] if shards else None


def pull(name: str, model_dir: str) -> int:
    os.makedirs(model_dir, exist_ok=True)
    path = resolve(name, model_dir)
    if path:
        print(path)
        return 0
    print(f"ie pull: '{name}' is not in {model_dir}.  This build does not download: copy the GGUF (all shards of a split file) "
          f"into that directory, or create a random-init checkpoint with `ie synth <preset> <out.gguf>`.", file=sys.stderr)
    return 1
