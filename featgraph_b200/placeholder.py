"""Shape carrier standing in for the reference's ``te.placeholder``.

The reference's ``build`` receives symbolic tensors whose only use is their static shape
and dtype (tests/test_module_spmm.py:18-19, python/featgraph/op/vanilla_spmm.py:37-38).
``build`` here accepts anything with a ``.shape`` (this class, a torch tensor, a numpy
array); ``placeholder`` exists so that call sites read the same.
"""


class Placeholder:
    def __init__(self, shape, dtype="float32", name="placeholder"):
        self.shape = tuple(int(s) for s in shape)
        self.dtype = str(dtype)
        self.name = name

    def __repr__(self):
        return "Placeholder(%s, shape=%s, dtype=%s)" % (self.name, self.shape, self.dtype)


def placeholder(shape, dtype="float32", name="placeholder"):
    return Placeholder(shape, dtype, name)


def static_shape(obj):
    """Shape tuple of a placeholder-like object (the reference's get_const_tuple)."""
    shape = getattr(obj, "shape", None)
    if shape is None:
        raise TypeError("expected an object with a .shape, got %r" % (type(obj),))
    return tuple(int(s) for s in shape)


def check_float32(obj):
    dt = getattr(obj, "dtype", "float32")
    name = str(dt).replace("torch.", "")
    if name != "float32":
        raise TypeError("only float32 features are supported, got %s" % (dt,))
