"""ctypes mirror of include/cc1d.h for tests that talk to libcc1d.so directly."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_PATH = os.path.join(ROOT, "causal_conv1d_b200", "libcc1d.so")
HEADER = os.path.join(ROOT, "include", "cc1d.h")

i32, i64, vp, sz = ctypes.c_int32, ctypes.c_int64, ctypes.c_void_p, ctypes.c_size_t
F32, F16, BF16 = 0, 1, 2


def _s3(name):
    return [(f"{name}_batch_stride", i64), (f"{name}_c_stride", i64), (f"{name}_l_stride", i64)]


class FwdParams(ctypes.Structure):
    _fields_ = ([("itype", i32), ("wtype", i32), ("width", i32), ("silu", i32),
                 ("batch", i64), ("dim", i64), ("seqlen", i64), ("x", vp)] + _s3("x") +
                [("weight", vp), ("weight_c_stride", i64), ("weight_width_stride", i64), ("bias", vp), ("out", vp)] +
                _s3("out") + [("seq_idx", vp), ("initial_states", vp)] + _s3("initial_states") +
                [("final_states", vp)] + _s3("final_states"))


class BwdParams(ctypes.Structure):
    _fields_ = ([("itype", i32), ("wtype", i32), ("width", i32), ("silu", i32),
                 ("batch", i64), ("dim", i64), ("seqlen", i64), ("x", vp)] + _s3("x") +
                [("weight", vp), ("weight_c_stride", i64), ("weight_width_stride", i64), ("bias", vp), ("dout", vp)] +
                _s3("dout") + [("dx", vp)] + _s3("dx") +
                [("dweight", vp), ("dweight_c_stride", i64), ("dweight_width_stride", i64), ("dbias", vp),
                 ("accumulate", i32), ("reserved0", i32), ("seq_idx", vp), ("initial_states", vp)] +
                _s3("initial_states") + [("dfinal_states", vp)] + _s3("dfinal_states") +
                [("dinitial_states", vp)] + _s3("dinitial_states") + [("workspace", vp), ("workspace_bytes", sz),
                                                                       ("peers", vp), ("phase", i32), ("reserved1", i32)])


class PeerGroup(ctypes.Structure):
    _fields_ = [("world", i32), ("rank", i32), ("capacity", i64), ("peer_base", vp * 16), ("status", vp),
                ("spin_limit", ctypes.c_uint32), ("reserved0", ctypes.c_uint32)]


class UpdateParams(ctypes.Structure):
    _fields_ = ([("itype", i32), ("wtype", i32), ("width", i32), ("silu", i32),
                 ("batch", i64), ("dim", i64), ("seqlen", i64), ("x", vp)] + _s3("x") +
                [("weight", vp), ("weight_c_stride", i64), ("weight_width_stride", i64), ("bias", vp), ("out", vp)] +
                _s3("out") + [("conv_state", vp), ("conv_state_len", i64)] + _s3("conv_state") +
                [("cache_seqlens", vp), ("conv_state_indices", vp)])


class VarlenParams(ctypes.Structure):
    _fields_ = [("itype", i32), ("cu_seqlens_is_int64", i32), ("total_tokens", i64), ("dim", i64), ("batch", i64),
                ("state_len", i64), ("x", vp), ("x_l_stride", i64), ("x_c_stride", i64), ("cu_seqlens", vp),
                ("states", vp), ("states_batch_stride", i64), ("states_c_stride", i64), ("states_l_stride", i64)]


class PrefillParams(ctypes.Structure):
    _fields_ = [("itype", i32), ("wtype", i32), ("width", i32), ("silu", i32),
                ("total_tokens", i64), ("dim", i64), ("nseq", i64), ("state_len", i64),
                ("x", vp), ("x_l_stride", i64),
                ("weight", vp), ("weight_c_stride", i64), ("weight_width_stride", i64), ("bias", vp),
                ("out", vp), ("out_l_stride", i64),
                ("seq_idx", vp), ("cu_seqlens", vp), ("state_indices", vp), ("has_initial_state", vp),
                ("initial_states", vp), ("initial_states_batch_stride", i64), ("initial_states_l_stride", i64),
                ("final_states", vp), ("final_states_batch_stride", i64), ("final_states_l_stride", i64)]


def declared_symbols():
    """Function names declared in include/cc1d.h."""
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(cc1d_[a-z0-9_]+)\s*\(", text)))


def load():
    lib = ctypes.CDLL(LIB_PATH)
    lib.cc1d_status_str.restype = ctypes.c_char_p
    lib.cc1d_status_str.argtypes = [ctypes.c_int]
    lib.cc1d_bwd_workspace_bytes.restype = sz
    lib.cc1d_bwd_workspace_bytes.argtypes = [ctypes.POINTER(BwdParams)]
    for name, st in (("cc1d_fwd", FwdParams), ("cc1d_bwd", BwdParams), ("cc1d_bwd_noalloc", BwdParams),
                     ("cc1d_update", UpdateParams),
                     ("cc1d_varlen_states", VarlenParams), ("cc1d_prefill_varlen", PrefillParams)):
        getattr(lib, name).argtypes = [ctypes.POINTER(st), vp]
        getattr(lib, name).restype = ctypes.c_int
    lib.cc1d_wait_expired.argtypes = []
    lib.cc1d_wait_expired.restype = ctypes.c_int
    lib.cc1d_seq_idx_from_cu_seqlens.argtypes = [vp, i64, i64, vp, vp]
    lib.cc1d_seq_idx_from_cu_seqlens.restype = ctypes.c_int
    return lib
