"""Element types with the names of the reference's singletons, plus the two 16-bit ones.

The reference defines ``float32 / int32 / int64`` as instances of ``Real`` / ``Int``
(kaleido/frontend/types.py:46-124), maps them to torch types (types.py:136-142) and back in
``Tensor.from_tensor`` (kaleido/frontend/tensor.py:122-130), and refuses everything else.  The
tensor-core kernels here compute on fp16 and bf16 storage, so those two exist here as well:
``float16`` and ``bfloat16`` (same width, told apart by ``brain``).
"""
import torch


class Number(object):
    def __init__(self, bits, signed=1):
        if bits not in (16, 32, 64):
            raise ValueError("the width should be 16, 32 or 64 bits")
        self.byte = bits  # the reference's name for the width in bits
        self.signed = signed

    def is_equal_type(self, other):
        return type(self) is type(other) and self.__dict__ == other.__dict__

    def __repr__(self):
        return "%s %s%d" % ("signed" if self.signed else "unsigned", type(self).__name__, self.byte)


class Int(Number):
    pass


class Real(Number):
    def __init__(self, bits, brain=False):
        super(Real, self).__init__(bits)
        if brain and bits != 16:
            raise ValueError("only the 16-bit type has a brain-float variant")
        self.brain = bool(brain)

    @property
    def max(self):
        return torch.finfo(internal_type_to_torch_type(self)).max

    def __repr__(self):
        return "signed %s%d" % ("BrainReal" if self.brain else "Real", self.byte)


float32 = Real(32)
float16 = Real(16)
bfloat16 = Real(16, brain=True)
int32 = Int(32)
int64 = Int(64)

_TO_TORCH = ((float32, torch.float32), (float16, torch.float16), (bfloat16, torch.bfloat16), (int32, torch.int32),
             (int64, torch.int64))
_FROM_STR = {"float": float32, "float32": float32, "half": float16, "float16": float16, "bfloat16": bfloat16,
             "int": int32, "int32": int32, "int64": int64}


def internal_type_to_torch_type(dtype):
    for mine, theirs in _TO_TORCH:
        if dtype is mine:
            return theirs
    raise NotImplementedError("no torch type for %r" % (dtype,))


def torch_type_to_internal_type(dtype):
    for mine, theirs in _TO_TORCH:
        if dtype is theirs:
            return mine
    raise NotImplementedError("no element type for %r" % (dtype,))


def str_to_internal_type(name):
    try:
        return _FROM_STR[name]
    except KeyError:
        raise NotImplementedError("unknown element type %r" % (name,))


def pytype_to_internal_type(x):
    if isinstance(x, bool):
        raise NotImplementedError()
    if isinstance(x, int):
        return int64
    if isinstance(x, float):
        return float32
    raise NotImplementedError()
