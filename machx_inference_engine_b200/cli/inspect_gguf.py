"""``ie inspect``: metadata and tensor listing of a GGUF file (the reference's tools/ie_inspect.cpp)."""
from __future__ import annotations

from collections import Counter

from ..formats.gguf import GGUFReader, type_name
from ..formats.model_config import ConfigError, read_config


def inspect(path: str, tensors: bool = False, out=None) -> int:
    import sys
    out = out or sys.stdout
    r = GGUFReader(path)
    print(f"file: {path}  (shards: {getattr(r, 'n_shards', 1)})", file=out)
    for k in sorted(r.kv):
        v = r.kv[k]
        if isinstance(v, (list, tuple)):
            v = f"[{len(v)} items] " + ", ".join(repr(x) for x in v[:4]) + (" ..." if len(v) > 4 else "")
        elif isinstance(v, str) and len(v) > 120:
            v = repr(v[:117] + "...")
        print(f"  {k} = {v}", file=out)
    by_type = Counter()
    total = 0
    for name, t in r.tensors.items():
        by_type[type_name(t.type)] += t.nbytes
        total += t.nbytes
        if tensors:
            print(f"  {name:48s} {type_name(t.type):6s} {'x'.join(str(d) for d in t.dims):>24s} {t.nbytes:>14,d} B", file=out)
    print(f"tensors: {len(r.tensors)}  payload: {total / 1e9:.3f} GB", file=out)
    for ty, nb in by_type.most_common():
        print(f"  {ty:6s} {nb / 1e9:10.3f} GB", file=out)
    try:
        c = read_config(r.kv, r.tensors.keys())
        print(f"config: arch={c.arch} layers={c.n_layers} hidden={c.hidden} heads={c.n_heads}/{c.n_kv_heads} head_dim={c.head_dim} "
              f"ffn={c.ffn} vocab={c.vocab} experts={c.n_experts}/{c.n_experts_used} ctx_train={c.ctx_train} template={c.template_family}", file=out)
    except ConfigError as e:
        print(f"config: not loadable ({e})", file=out)
    return 0
