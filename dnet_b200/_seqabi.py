"""ctypes binding of libdnet_b200_seq.so (include/dnet_b200_seq.h): the batched step of models built from
sequence mixers.  Built in-tree on first use; no CPU fallback -- every call checks its return code."""
from __future__ import annotations

import ctypes as C
import os
import re
from pathlib import Path
from typing import List

from dnet_b200._cabi import DnError

_ROOT = Path(__file__).resolve().parent
HEADER_PATH = _ROOT.parent / "include" / "dnet_b200_seq.h"

DN_SEQ_BF16, DN_SEQ_F32 = 0, 1
DN_MIX_ATTENTION, DN_MIX_DELTA = 0, 1
# dn_seq_bind slots, in the header's order
_LAYER_SLOTS = ["norm1", "norm2", "mix.q", "mix.k", "mix.v", "mix.o", "mix.q.conv", "mix.k.conv", "mix.v.conv", "mix.q.norm",
                "mix.k.norm", "mix.a", "mix.b", "mix.g", "mix.A_log", "mix.dt_bias", "mix.norm", "mlp.gate", "mlp.up", "mlp.down",
                "hc1.in", "hc1.out", "hc1.mix", "hc2.in", "hc2.out", "hc2.mix"]
LAYER_SLOT = {n: i for i, n in enumerate(_LAYER_SLOTS)}
MODEL_SLOT = {"embed": 100, "final.norm": 101, "head": 102}
# phases of a step, in the header's order (dn_seq_profile_read)
PHASES = ["embed", "norm", "proj", "attn_prep", "attn", "delta_prep", "delta_rule", "delta_out", "conv_carry", "out_proj",
          "write_back", "ff_up", "ff_down", "head", "other"]


class LayerCfg(C.Structure):
    _fields_ = [("mixer", C.c_int32), ("heads", C.c_int32), ("kv_heads", C.c_int32), ("dim", C.c_int32), ("vdim", C.c_int32),
                ("conv", C.c_int32), ("chunk", C.c_int32), ("rot_dims", C.c_int32), ("rot_base", C.c_float), ("scale", C.c_float),
                ("kv_from", C.c_int32), ("ff", C.c_int32)]


class SeqCfg(C.Structure):
    _fields_ = [("width", C.c_int32), ("vocab", C.c_int32), ("n_layers", C.c_int32), ("streams", C.c_int32), ("dtype", C.c_int32),
                ("eps", C.c_float), ("embed_scale", C.c_float), ("pool_pages", C.c_int32), ("max_seqs", C.c_int32),
                ("max_batch_tokens", C.c_int32)]


def declared_symbols() -> List[str]:
    txt = re.sub(r"/\*.*?\*/", "", HEADER_PATH.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(dn_seq_[a-z0-9_]+)\s*\(", txt)))


_vp, _i = C.c_void_p, C.c_int
_I32P = C.POINTER(C.c_int32)
_PROTOS = {
    "dn_seq_init": (_i, [_i]),
    "dn_seq_last_error": (C.c_char_p, []),
    "dn_seq_launch_count": (C.c_int64, []),
    "dn_seq_model_create": (_i, [C.POINTER(SeqCfg), C.POINTER(LayerCfg), C.POINTER(_vp)]),
    "dn_seq_model_destroy": (_i, [_vp]),
    "dn_seq_bind": (_i, [_vp, _i, _i, _vp]),
    "dn_seq_open": (_i, [_vp, _vp, C.POINTER(_i)]),
    "dn_seq_close": (_i, [_vp, _i]),
    "dn_seq_length": (_i, [_vp, _i]),
    "dn_seq_free_pages": (_i, [_vp]),
    "dn_seq_free_slots": (_i, [_vp]),
    "dn_seq_check": (_i, [_vp, _vp]),
    "dn_seq_profile": (_i, [_vp, _i]),
    "dn_seq_profile_read": (_i, [_vp, C.POINTER(C.c_double), _i]),
    "dn_seq_set_graphs": (_i, [_vp, _i]),
    "dn_seq_step": (_i, [_vp, _i, _I32P, _I32P, _I32P, _i, _I32P, _vp, _vp, _vp]),
}
_lib = None


def load() -> C.CDLL:
    global _lib
    if _lib is None:
        path = os.environ.get("DNET_B200_SEQ_LIB")
        if not path:
            from dnet_b200 import build as b

            path = str(b.build_seq())
        lib = C.CDLL(path)
        for name, (res, args) in _PROTOS.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def check(rc: int) -> int:
    if rc < 0:
        raise DnError(rc, load().dn_seq_last_error().decode("utf-8", "replace"))
    return rc


_inited = set()


def init(device: int) -> None:
    if device not in _inited:
        check(load().dn_seq_init(int(device)))
        _inited.add(device)
