"""Bindings of the hand-written sm_100a kernels (placeholder until the extension is loaded)."""


def install():
    raise RuntimeError("q38.ops: the CUDA extension is not built; run `python -c 'import __graft_entry__ as g; g.build()'`")
