"""Stand-ins for the reference's four PyTorch extension modules, on this library's kernels.

Put this folder on ``sys.path`` (``sys.path.insert(0, niti_b200.compat.path())``) and the reference's
unmodified ``ti_torch.py`` finds ``cutlassconv_cuda``, ``int8mm_cuda``, ``int8pool_cuda`` and
``int8conv_cuda`` here, with the signatures of its pybind11 modules (cutlassconv.cpp:57-73, int8mm.cpp:9-18,
int8pool.cpp, int8conv.cpp:35-45): tensors in, a freshly allocated tensor out, ``RuntimeError`` for a tensor
that is not on the GPU or not contiguous.  The modules call the C ABI (``niti_b200.ops``); there is no CPU path.
"""
import os


def path():
    """The directory to put on sys.path so that `import cutlassconv_cuda` (etc.) resolves to these modules."""
    return os.path.dirname(os.path.abspath(__file__))


def check_input(*tensors):
    """CHECK_INPUT of the reference's bindings (e.g. cutlassconv.cpp:43-45)."""
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError("must be a CUDA tensor")
        if not t.is_contiguous():
            raise RuntimeError("must be contiguous")
