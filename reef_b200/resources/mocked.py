"""The reference's two-kernel known-answer model (reference:
resource/mocked_kernel/mocked_kernel.json:1-72, mocked_kernel.cu:9-29):
``temp = a[t] + b[i]`` then ``output = temp[t] * c[i]`` with ``t = i % 128`` —
the first operand is indexed by the thread offset only.  With every input equal
to 3 every output is 18 (reference: src/reef/test/test.cpp:102-116)."""
from .graph import Graph


def build_mocked_kernel() -> Graph:
    g = Graph("mocked_kernel")
    a = g.input("a", 8192)
    b = g.input("b", 8192)
    temp = g.add_storage("temp", 8192)
    c = g.input("c", 8192)
    out = g.add_storage("output", 8192)
    g.kernel("add", [b, a, temp])
    g.kernel("multiply", [temp, c, out])
    return g
