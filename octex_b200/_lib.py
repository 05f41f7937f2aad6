"""ctypes binding of liboctex_b200.so (the C interface in include/octex_b200.h).

There is no fallback: when the shared library is missing or cannot be loaded, every use raises.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
#: the library built in-tree; OCTEX_B200_LIB names another build of it (a debug or experimental one)
LIB_PATH = os.environ.get("OCTEX_B200_LIB") or os.path.join(_PKG, "lib", "liboctex_b200.so")
CUVS_ERROR, CUVS_SUCCESS = 0, 1
_lib = None


class SearchParams(C.Structure):
    """struct cuvsOctexSearchParams"""
    _fields_ = [("read", C.c_int32), ("starts", C.c_int32), ("waves", C.c_int32),
                ("rerank", C.c_int32), ("wave_rerank", C.c_int32), ("batch", C.c_int32),
                ("sketch_rank", C.c_bool), ("final_rerank", C.c_int32),
                ("balanced_gather", C.c_bool), ("fused_merge", C.c_bool), ("use_graph", C.c_bool)]


class LoadParams(C.Structure):
    """struct cuvsOctexLoadParams"""
    _fields_ = [("devices", C.POINTER(C.c_int32)), ("n_devices", C.c_int32),
                ("placement", C.c_int32), ("vectors_on_host", C.c_bool),
                ("shard_vectors", C.c_bool), ("table_on_host", C.c_bool), ("sketch", C.c_int32),
                ("parts", C.c_int32), ("copies_per_part", C.c_int32), ("copies_limit", C.c_int32),
                ("list_limit", C.c_int32)]


class IndexParams(C.Structure):
    """struct cuvsOctexIndexParams"""
    _fields_ = [("copies", C.c_int32), ("blocks", C.c_int32), ("pca_dims", C.c_int32),
                ("spacings", C.POINTER(C.c_float)), ("n_spacings", C.c_int32),
                ("list_len", C.c_int32), ("min_cell", C.c_int32), ("log_buckets", C.c_int32),
                ("sketch_width", C.c_int32), ("table_len", C.c_int32),
                ("reverse_edges", C.c_bool), ("exact_lists", C.c_bool), ("list_probes", C.c_int32),
                ("member_lists", C.c_bool), ("exact_table_max", C.c_int64),
                ("table_passes", C.c_int32), ("table_sketch_order", C.c_bool),
                ("write_behind", C.c_bool), ("seed", C.c_uint64),
                ("devices", C.POINTER(C.c_int32)), ("n_devices", C.c_int32)]


class IndexHandle(C.Structure):
    """cuvsOctexIndex"""
    _fields_ = [("addr", C.c_size_t)]


class Arrays(C.Structure):
    """octexB200Arrays"""
    _fields_ = [("n", C.c_int64), ("dim", C.c_int64), ("copies", C.c_int32), ("blocks", C.c_int32),
                ("list_len", C.c_int32), ("log_buckets", C.c_int32), ("sketch_width", C.c_int32),
                ("table_len", C.c_int32), ("spacings", C.c_void_p), ("n_spacings", C.c_int32),
                ("borrow", C.c_int32), ("stride", C.c_int64), ("mmax", C.c_int64),
                ("mean", C.c_void_p), ("proj", C.c_void_p), ("shift", C.c_void_p),
                ("lists", C.c_void_p), ("keys", C.c_void_p), ("offsets", C.c_void_p),
                ("base", C.c_void_p), ("sketch_basis", C.c_void_p), ("sketch_scale", C.c_void_p),
                ("sketch", C.c_void_p), ("vectors", C.c_void_p), ("table", C.c_void_p)]


class DLDevice(C.Structure):
    _fields_ = [("device_type", C.c_int32), ("device_id", C.c_int32)]


class DLDataType(C.Structure):
    _fields_ = [("code", C.c_uint8), ("bits", C.c_uint8), ("lanes", C.c_uint16)]


class DLTensor(C.Structure):
    _fields_ = [("data", C.c_void_p), ("device", DLDevice), ("ndim", C.c_int32),
                ("dtype", DLDataType), ("shape", C.POINTER(C.c_int64)),
                ("strides", C.POINTER(C.c_int64)), ("byte_offset", C.c_uint64)]


class DLManagedTensor(C.Structure):
    _fields_ = [("dl_tensor", DLTensor), ("manager_ctx", C.c_void_p), ("deleter", C.c_void_p)]


#: every symbol include/octex_b200.h declares
SYMBOLS = (
    "cuvsResourcesCreate", "cuvsResourcesDestroy", "cuvsStreamSet", "cuvsStreamGet",
    "cuvsStreamSync", "cuvsGetLastErrorText", "cuvsSetLastErrorText",
    "cuvsOctexIndexParamsCreate", "cuvsOctexIndexParamsDestroy", "cuvsOctexLoadParamsCreate",
    "cuvsOctexLoadParamsDestroy", "cuvsOctexSearchParamsCreate", "cuvsOctexSearchParamsDestroy",
    "cuvsOctexIndexCreate", "cuvsOctexIndexDestroy", "cuvsOctexIndexGetSize",
    "cuvsOctexIndexGetDim", "cuvsOctexIndexGetCopies", "cuvsOctexIndexGetNumDevices",
    "cuvsOctexIndexGetDevices", "cuvsOctexIndexGetDeviceBytes", "cuvsOctexBuild", "cuvsOctexLoad",
    "cuvsOctexSearch", "octexB200Search", "octexB200LoadRank", "octexB200Attach",
    "octexB200SearchResident", "octexB200ProfileBatch", "octexB200SetDebug", "octexB200Fetch",
    "octexB200CellCodes", "octexB200QueryCodesStatic", "octexB200SetProjection",
    "octexB200CommUniqueId", "octexB200CommInit", "octexB200CommDisconnect", "octexB200CheckLast",
    "octexB200MemoryReport", "octexB200Build", "octexB200ExactNeighbors", "octexB200SetTable", "octexB200SearchedTable",
)


def lib():
    """The loaded library; raises ImportError when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"octex_b200: {LIB_PATH} is missing; build it with "
                "`python -c 'import __graft_entry__ as g; g.build()'` (needs nvcc). "
                "There is no CPU fallback.")
        L = C.CDLL(LIB_PATH)
        L.cuvsGetLastErrorText.restype = C.c_char_p
        L.cuvsSetLastErrorText.restype = None
        _lib = L
    return _lib


def check(rc: int):
    if rc != CUVS_SUCCESS:
        text = lib().cuvsGetLastErrorText()
        msg = text.decode() if text else "octex: unknown error"
        if "CUDA error" in msg:
            raise RuntimeError(msg)
        raise ValueError(msg)
