"""ctypes binding of the C ABI in ``include/mk_abi.h``.

Same contract as the reference's ``sgl_muse_mega/common/host.py:21-187``: the header is the only place a bind field is
declared (the ctypes mirrors are generated from it), ``make`` demands every field by name, a ``Library`` wraps the
shared object, a ``Module`` a device binding and a ``Launch`` a bound launch record whose call enqueues it.
There is no fallback: a missing or unloadable library raises.
"""

from __future__ import annotations

import ctypes
import os
import re
import weakref
from pathlib import Path

HEADER = Path(__file__).resolve().parent.parent.parent / "include" / "mk_abi.h"

_SCALARS = {"uint64_t": ctypes.c_uint64, "int64_t": ctypes.c_int64, "double": ctypes.c_double}
_FIELD = re.compile(r"(uint64_t|int64_t|double)\s+(\w+)\s*(?:\[\s*(\w+)\s*\])?\s*;")


def parse_header(path: Path = HEADER) -> tuple[dict, dict]:
    """-> ({struct name: ctypes.Structure subclass}, {macro: int}) from the ABI header."""
    text = path.read_text()
    macros = {k: int(v) for k, v in re.findall(r"^#define\s+(\w+)\s+(\d+)\s*$", text, re.M)}
    structs = {}
    for body, name in re.findall(r"typedef struct \w+ \{(.*?)\}\s*(\w+);", text, re.S):
        fields = []
        for raw in body.splitlines():
            line = raw.split("//")[0].strip()
            if not line:
                continue
            m = _FIELD.fullmatch(line)
            if m is None:
                raise ValueError(f"{path.name}: cannot parse field of {name}: {line!r}")
            ctype = _SCALARS[m[1]]
            if m[3]:
                ctype = ctype * (int(m[3]) if m[3].isdigit() else macros[m[3]])
            fields.append((m[2], ctype))
        structs[name] = type(name, (ctypes.Structure,), {"_fields_": fields})
    return structs, macros


STRUCTS, MACROS = parse_header()


def _value(v):
    if v is None:
        return 0
    if hasattr(v, "data_ptr"):
        return v.data_ptr()
    return v


def make(struct: str, **values) -> ctypes.Structure:
    """A bind struct with every field given by name (tensors as their data pointers, None as 0). ``*_peer`` arrays may
    be given shorter than their capacity; the rest stays 0."""
    cls = STRUCTS[struct]
    names = [n for n, _ in cls._fields_]
    missing, unknown = set(names) - set(values), set(values) - set(names)
    if missing or unknown:
        raise ValueError(f"{struct}: missing {sorted(missing)}, unknown {sorted(unknown)}")
    out = cls()
    for name, ctype in cls._fields_:
        v = values[name]
        if issubclass(ctype, ctypes.Array):
            if len(v) > ctype._length_:
                raise ValueError(f"{struct}.{name}: {len(v)} entries exceed {ctype._length_}")
            setattr(out, name, ctype(*[_value(x) for x in v]))
        else:
            setattr(out, name, _value(v))
    return out


SYMM_HANDLE_BYTES = 64  # MK_SYMM_HANDLE_BYTES


EXPORTS = (
    "mk_last_error", "mk_module_load", "mk_module_free", "mk_launch", "mk_launch_step", "mk_launch_free",
    "mk_launch_info", "mk_launch_params", "mk_launch_status", "mk_layer_constants", "mk_layer_bind", "mk_qkv_constants", "mk_qkv_bind",
    "mk_qkv_launch_static", "mk_feeds_bind", "mk_entry_bind", "mk_lm_head_bind", "mk_softcap_bind", "mk_accept_bind",
    "mk_symm_alloc", "mk_symm_open", "mk_symm_close", "mk_symm_free", "mk_dflash_constants", "mk_dflash_entry_bind",
    "mk_dflash_layer_bind", "mk_dflash_draft_head_bind", "mk_dflash_kv_sync_bind", "mk_dflash_tree_bind",
    "mk_dflash_tree_compact_bind",
)  # fmt: skip


class Library:
    """The shared library, loaded RTLD_LOCAL (as reference host.py:85-90)."""

    def __init__(self, path: Path):
        self.path = Path(path)
        if not self.path.exists():
            raise FileNotFoundError(f"{self.path}: build it with `python -m sgl_muse_mega_b200.common.build`")
        self.dll = ctypes.CDLL(str(self.path), mode=os.RTLD_LOCAL)
        d, vp, P = self.dll, ctypes.c_void_p, ctypes.POINTER
        d.mk_last_error.restype = ctypes.c_char_p
        d.mk_module_load.argtypes = [vp, ctypes.c_uint64, ctypes.c_char_p, P(vp)]
        d.mk_module_free.argtypes = [vp]
        d.mk_module_free.restype = None
        d.mk_launch.argtypes = [vp, ctypes.c_uint64, ctypes.c_int]
        d.mk_launch_step.argtypes = [vp, ctypes.c_uint64, ctypes.c_int64, ctypes.c_int64]
        d.mk_launch_free.argtypes = [vp]
        d.mk_launch_free.restype = None
        d.mk_launch_info.argtypes = [vp, P(STRUCTS["MkLaunchInfo"])]
        d.mk_launch_params.argtypes = [vp, ctypes.c_char_p, ctypes.c_uint64]
        d.mk_launch_status.argtypes = [vp, ctypes.c_uint64, P(STRUCTS["MkLaunchStatus"])]
        d.mk_layer_constants.argtypes = [P(STRUCTS["MkLayerShape"]), P(STRUCTS["MkLayerConstants"])]
        d.mk_layer_bind.argtypes = [vp, P(STRUCTS["MkLayerShape"]), P(STRUCTS["MkLayerBind"]), P(vp)]
        d.mk_qkv_constants.argtypes = [P(STRUCTS["MkQkvBind"]), P(STRUCTS["MkQkvConstants"])]
        d.mk_qkv_bind.argtypes = [vp, P(STRUCTS["MkQkvBind"]), P(vp)]
        d.mk_qkv_launch_static.argtypes = [P(STRUCTS["MkQkvBind"]), ctypes.c_uint64]
        for fn, st in (("mk_feeds_bind", "MkFeedsBind"), ("mk_entry_bind", "MkEntryBind"), ("mk_lm_head_bind", "MkLmHeadBind"),
                       ("mk_softcap_bind", "MkSoftcapBind"), ("mk_accept_bind", "MkAcceptBind")):  # fmt: skip
            getattr(d, fn).argtypes = [vp, P(STRUCTS[st]), P(vp)]
        d.mk_dflash_constants.argtypes = [P(STRUCTS["MkDflashShape"]), P(STRUCTS["MkDflashConstants"])]
        for fn, st in (("mk_dflash_entry_bind", "MkDflashEntryBind"), ("mk_dflash_layer_bind", "MkDflashLayerBind"),
                       ("mk_dflash_draft_head_bind", "MkDflashDraftHeadBind")):  # fmt: skip
            getattr(d, fn).argtypes = [vp, P(STRUCTS["MkDflashShape"]), P(STRUCTS[st]), P(vp)]
        d.mk_dflash_kv_sync_bind.argtypes = [vp, P(STRUCTS["MkDflashKvSyncBind"]), P(vp)]
        d.mk_dflash_tree_bind.argtypes = [vp, P(STRUCTS["MkDflashTreeBind"]), P(vp)]
        d.mk_dflash_tree_compact_bind.argtypes = [vp, P(STRUCTS["MkDflashTreeCompactBind"]), P(vp)]
        d.mk_symm_alloc.argtypes = [ctypes.c_int64, P(ctypes.c_uint64), ctypes.c_char_p]
        d.mk_symm_open.argtypes = [ctypes.c_char_p, P(ctypes.c_uint64)]
        d.mk_symm_close.argtypes = [ctypes.c_uint64]
        d.mk_symm_free.argtypes = [ctypes.c_uint64]

    def check(self, rc: int, what: str) -> None:
        if rc != 0:
            raise RuntimeError(f"{self.path.name}: {what}: {self.dll.mk_last_error().decode()}")

    def load(self) -> "Module":
        """Binds the built-in kernels to the current CUDA device."""
        out = ctypes.c_void_p()
        self.check(self.dll.mk_module_load(None, 0, None, ctypes.byref(out)), "mk_module_load")
        return Module(self, out)

    def layer_constants(self, shape) -> ctypes.Structure:
        c = STRUCTS["MkLayerConstants"]()
        self.check(self.dll.mk_layer_constants(ctypes.byref(shape), ctypes.byref(c)), "mk_layer_constants")
        return c

    def layer_bind(self, module: "Module | None", shape, bind) -> "Launch":
        """``module`` None gives a pack-only record: validated, cannot launch (as reference abi.h:38-39)."""
        out = ctypes.c_void_p()
        self.check(
            self.dll.mk_layer_bind(module.handle if module else None, ctypes.byref(shape), ctypes.byref(bind), ctypes.byref(out)),
            "mk_layer_bind",
        )
        return Launch(self, out, module)


    def qkv_constants(self, bind) -> ctypes.Structure:
        c = STRUCTS["MkQkvConstants"]()
        self.check(self.dll.mk_qkv_constants(ctypes.byref(bind), ctypes.byref(c)), "mk_qkv_constants")
        return c

    def qkv_bind(self, module: "Module | None", bind) -> "Launch":
        out = ctypes.c_void_p()
        self.check(self.dll.mk_qkv_bind(module.handle if module else None, ctypes.byref(bind), ctypes.byref(out)), "mk_qkv_bind")
        return Launch(self, out, module)


    def bind(self, fn_name: str, module: "Module | None", bind) -> "Launch":
        """Any ``mk_*_bind(module, bind, out)`` entry point by name (feeds, entry, lm_head, softcap, accept)."""
        out = ctypes.c_void_p()
        fn = getattr(self.dll, fn_name)
        self.check(fn(module.handle if module else None, ctypes.byref(bind), ctypes.byref(out)), fn_name)
        return Launch(self, out, module)


    def dflash_constants(self, shape) -> ctypes.Structure:
        c = STRUCTS["MkDflashConstants"]()
        self.check(self.dll.mk_dflash_constants(ctypes.byref(shape), ctypes.byref(c)), "mk_dflash_constants")
        return c

    def dflash_bind(self, fn_name: str, module: "Module | None", shape, bind) -> "Launch":
        """``mk_dflash_{entry,layer,draft_head}_bind(module, shape, bind, out)`` by name."""
        out = ctypes.c_void_p()
        fn = getattr(self.dll, fn_name)
        self.check(fn(module.handle if module else None, ctypes.byref(shape), ctypes.byref(bind), ctypes.byref(out)), fn_name)
        return Launch(self, out, module)

    # ---- memory shared between the ranks' processes ----
    def symm_alloc(self, nbytes: int) -> tuple[int, bytes]:
        """(device pointer, 64-byte handle) of zeroed memory on the current device that peer processes can map."""
        ptr, handle = ctypes.c_uint64(), ctypes.create_string_buffer(SYMM_HANDLE_BYTES)
        self.check(self.dll.mk_symm_alloc(nbytes, ctypes.byref(ptr), handle), "mk_symm_alloc")
        return ptr.value, handle.raw

    def symm_open(self, handle: bytes) -> int:
        ptr = ctypes.c_uint64()
        self.check(self.dll.mk_symm_open(handle, ctypes.byref(ptr)), "mk_symm_open")
        return ptr.value

    def symm_close(self, ptr: int) -> None:
        self.check(self.dll.mk_symm_close(ptr), "mk_symm_close")

    def symm_free(self, ptr: int) -> None:
        self.check(self.dll.mk_symm_free(ptr), "mk_symm_free")


def _free_with(obj, fn, handle) -> None:
    weakref.finalize(obj, fn, handle).atexit = False


class Module:
    def __init__(self, lib: Library, handle):
        self.lib, self.handle = lib, handle
        _free_with(self, lib.dll.mk_module_free, handle)


class Launch:
    def __init__(self, lib: Library, handle, module):
        self.lib, self.handle, self.module = lib, handle, module
        _free_with(self, lib.dll.mk_launch_free, handle)

    def __call__(self, stream: int, pdl: bool = False) -> None:
        self.lib.check(self.lib.dll.mk_launch(self.handle, stream, int(pdl)), "mk_launch")

    def step(self, stream: int, first: int, count: int) -> None:
        self.lib.check(self.lib.dll.mk_launch_step(self.handle, stream, first, count), "mk_launch_step")

    def info(self) -> ctypes.Structure:
        i = STRUCTS["MkLaunchInfo"]()
        self.lib.check(self.lib.dll.mk_launch_info(self.handle, ctypes.byref(i)), "mk_launch_info")
        return i

    def params(self) -> dict:
        """What a layer bind wired between its kernels (``mk_launch_params``): {"post_norm.wait": {"wait": "packets",
        "present": 3, ...}, "o_proj.signal": {"signal": 0, ...}, ...}; works on pack-only records."""
        buf = ctypes.create_string_buffer(4096)
        n = self.lib.dll.mk_launch_params(self.handle, buf, len(buf))
        self.lib.check(0 if n >= 0 else -1, "mk_launch_params")
        out = {}
        for line in buf.value.decode().splitlines():
            name, *pairs = line.split()
            fields = dict(p.split("=", 1) for p in pairs)
            kind = "wait" if "wait" in fields else "signal" if "signal" in fields else "stages"
            out[name if kind == "stages" else f"{name}.{kind}"] = {k: (v if k == "wait" else int(v, 0)) for k, v in fields.items()}
        return out

    def status(self, stream: int) -> ctypes.Structure:
        s = STRUCTS["MkLaunchStatus"]()
        self.lib.check(self.lib.dll.mk_launch_status(self.handle, stream, ctypes.byref(s)), "mk_launch_status")
        return s


_LIB: Library | None = None


def library() -> Library:
    """The process-wide library handle (built in-tree on first use if stale)."""
    global _LIB
    if _LIB is None:
        from . import build

        _LIB = Library(build.build())
    return _LIB
