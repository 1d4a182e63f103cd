"""Python binding of the URMA API (libumdk_urma.so) through its flat convenience layer.

    ctx = urma.Context("shm0")
    ep = ctx.endpoint(depth=256, recv_token=7)
    seg = ctx.register(buffer_tensor_or_ctypes_array, access=urma.READ | urma.WRITE | urma.ATOMIC, token=42)
    # exchange ep.blob and seg.blob with the peer over any side channel (e.g. torch.distributed)
    peer = ctx.import_endpoint(peer_ep_blob, token=7); rseg = ctx.import_segment(peer_seg_blob, token=42)
    ep.write(peer, rseg, rseg.va + off, local_addr, nbytes); ep.wait(1)
    old = ep.fetch_add(peer, rseg, rseg.va, 1)

Same object model as the reference's sample (src/urma/examples/urma_sample.c): context, jetty, segment, import,
one-sided / two-sided / atomic verbs, completion polling.
"""
from __future__ import annotations

import ctypes
import struct
from typing import List, Optional, Tuple

from . import _native

LOCAL_ONLY, READ, WRITE, ATOMIC = 1, 2, 4, 8
OPC_WRITE, OPC_WRITE_IMM, OPC_READ = 0x00, 0x01, 0x10
OPC_CAS, OPC_SWAP, OPC_FADD, OPC_FSUB, OPC_FAND, OPC_FOR, OPC_FXOR = 0x20, 0x21, 0x22, 0x23, 0x24, 0x25, 0x26
OPC_SEND, OPC_SEND_IMM, OPC_NOP = 0x40, 0x41, 0x51
CR_SUCCESS, CR_REM_ACCESS_ABORT, CR_ACK_TIMEOUT, CR_FLUSH = 0, 8, 9, 11
CR_RNR = 10        # URMA_CR_RNR_RETRY_CNT_EXC_ERR: the target had no receive buffer posted
CR_FLAG_RECV = 1   # Completion.flag bit: receive-side completion
SEG_BLOB, JETTY_BLOB = 64, 32


class UrmaError(RuntimeError):
    pass


def _lib():
    lib = _native.urma()
    if getattr(lib, "_umdk_typed", False):
        return lib
    vp = ctypes.c_void_p
    lib.urma_simple_open.restype = vp
    lib.urma_simple_open.argtypes = [ctypes.c_char_p]
    lib.urma_simple_close.argtypes = [vp]
    lib.urma_simple_ep_create.restype = vp
    lib.urma_simple_ep_create.argtypes = [vp, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_int]
    lib.urma_simple_ep_destroy.argtypes = [vp]
    lib.urma_simple_ep_blob.argtypes = [vp, ctypes.c_char_p]
    lib.urma_simple_ep_import.restype = vp
    lib.urma_simple_ep_import.argtypes = [vp, ctypes.c_char_p, ctypes.c_uint32]
    lib.urma_simple_seg_register.restype = vp
    lib.urma_simple_seg_register.argtypes = [vp, vp, ctypes.c_uint64, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_char_p]
    lib.urma_simple_seg_import.restype = vp
    lib.urma_simple_seg_import.argtypes = [vp, ctypes.c_char_p, ctypes.c_uint32]
    lib.urma_simple_post.argtypes = [vp, vp, ctypes.c_int, vp, ctypes.c_uint64, vp, ctypes.c_uint64, ctypes.c_uint32,
                                     ctypes.c_uint64, ctypes.c_uint64, ctypes.c_int]
    lib.urma_simple_atomic.argtypes = [vp, vp, ctypes.c_int, vp, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_uint64,
                                       vp, ctypes.c_uint64]
    lib.urma_simple_post_recv.argtypes = [vp, vp, ctypes.c_uint32, ctypes.c_uint64]
    lib.urma_simple_wait.argtypes = [vp, ctypes.c_int, ctypes.c_int, ctypes.c_int, vp, vp, vp, vp, vp]
    lib.urma_simple_poll.argtypes = [vp, ctypes.c_int, vp, vp, vp, vp, vp]
    lib.urma_unregister_seg.argtypes = [vp]
    lib.urma_unimport_seg.argtypes = [vp]
    lib.urma_unimport_jetty.argtypes = [vp]
    lib._umdk_typed = True
    return lib


def _addr_len(buf) -> Tuple[int, int]:
    """(address, nbytes) of a torch CPU tensor, numpy array, ctypes array or (addr, len) tuple."""
    if isinstance(buf, tuple):
        return int(buf[0]), int(buf[1])
    if hasattr(buf, "data_ptr"):
        return buf.data_ptr(), buf.numel() * buf.element_size()
    if hasattr(buf, "ctypes") and hasattr(buf, "nbytes"):
        return buf.ctypes.data, buf.nbytes
    return ctypes.addressof(buf), ctypes.sizeof(buf)


class Segment:
    def __init__(self, ctx: "Context", handle: int, blob: bytes, imported: bool, keep=None):
        self.ctx, self.handle, self.blob, self.imported, self._keep = ctx, handle, blob, imported, keep
        # urma_seg_t: eid[16], uasid u32, (pad) va u64, len u64, attr u32, token_id u32
        self.uasid, self.va, self.len, self.attr, self.token_id = struct.unpack_from("<I4xQQII", blob, 16)

    def close(self):
        if self.handle:
            (self.ctx.lib.urma_unimport_seg if self.imported else self.ctx.lib.urma_unregister_seg)(self.handle)
            self.handle = 0


class Completion(tuple):
    """(status, user_ctx, length, imm, flag)"""
    status = property(lambda s: s[0])
    user_ctx = property(lambda s: s[1])
    length = property(lambda s: s[2])
    imm = property(lambda s: s[3])
    flags = property(lambda s: s[4])
    is_recv = property(lambda s: bool(s[4] & 1))


class Endpoint:
    def __init__(self, ctx: "Context", depth: int, recv_token: int, interrupt: bool):
        self.ctx = ctx
        self.lib = ctx.lib
        self.handle = self.lib.urma_simple_ep_create(ctx.handle, depth, recv_token, int(interrupt))
        if not self.handle:
            raise UrmaError("urma_simple_ep_create failed")
        b = ctypes.create_string_buffer(JETTY_BLOB)
        self.lib.urma_simple_ep_blob(self.handle, b)
        self.blob = bytes(b.raw)
        self._result = ctypes.c_uint64(0)

    def _post(self, peer, opc, rseg, raddr, laddr, n, imm=0, user_ctx=0, signaled=True):
        rc = self.lib.urma_simple_post(self.handle, peer, opc, rseg.handle if rseg else None, raddr, None, laddr, n,
                                       imm, user_ctx, int(signaled))
        if rc != 0:
            raise UrmaError(f"post opcode 0x{opc:x} failed: {rc}")

    def write(self, peer, rseg: Segment, raddr: int, laddr: int, n: int, user_ctx=0, signaled=True, imm=None):
        self._post(peer, OPC_WRITE if imm is None else OPC_WRITE_IMM, rseg, raddr, laddr, n, imm or 0, user_ctx, signaled)

    def read(self, peer, rseg: Segment, raddr: int, laddr: int, n: int, user_ctx=0):
        self._post(peer, OPC_READ, rseg, raddr, laddr, n, 0, user_ctx, True)

    def send(self, peer, laddr: int, n: int, user_ctx=0, imm=None):
        self._post(peer, OPC_SEND if imm is None else OPC_SEND_IMM, None, 0, laddr, n, imm or 0, user_ctx, True)

    def post_recv(self, buf, user_ctx=0):
        a, n = _addr_len(buf)
        rc = self.lib.urma_simple_post_recv(self.handle, a, n, user_ctx)
        if rc != 0:
            raise UrmaError(f"post_recv failed: {rc}")

    def atomic(self, peer, opc, rseg: Segment, raddr: int, operand: int, compare: int = 0, result_addr: int = 0,
               user_ctx=0):
        rc = self.lib.urma_simple_atomic(self.handle, peer, opc, rseg.handle, raddr, operand & (2 ** 64 - 1),
                                         compare & (2 ** 64 - 1), result_addr or None, user_ctx)
        if rc != 0:
            raise UrmaError(f"atomic opcode 0x{opc:x} failed: {rc}")

    def fetch_add(self, peer, rseg: Segment, raddr: int, value: int, timeout_ms=5000) -> int:
        """Blocking fetch-and-add; returns the old value."""
        self.atomic(peer, OPC_FADD, rseg, raddr, value, 0, ctypes.addressof(self._result))
        self.wait(1, timeout_ms)
        return self._result.value

    def compare_swap(self, peer, rseg: Segment, raddr: int, compare: int, swap: int, timeout_ms=5000) -> int:
        self.atomic(peer, OPC_CAS, rseg, raddr, swap, compare, ctypes.addressof(self._result))
        self.wait(1, timeout_ms)
        return self._result.value

    def poll(self, max_n=16) -> List[Completion]:
        return self._collect(self.lib.urma_simple_poll, max_n)

    def wait(self, want=1, timeout_ms=5000, check=True) -> List[Completion]:
        st = (ctypes.c_int * want)()
        uc = (ctypes.c_uint64 * want)()
        ln = (ctypes.c_uint32 * want)()
        im = (ctypes.c_uint64 * want)()
        fl = (ctypes.c_uint32 * want)()
        n = self.lib.urma_simple_wait(self.handle, want, timeout_ms, want, st, uc, ln, im, fl)
        out = [Completion((st[i], uc[i], ln[i], im[i], fl[i])) for i in range(max(n, 0))]
        if check:
            if n < want:
                raise UrmaError(f"timed out waiting for {want} completions (got {n})")
            bad = [c for c in out if c.status != CR_SUCCESS]
            if bad:
                raise UrmaError(f"completion with error status {bad[0].status}")
        return out

    def recover(self) -> int:
        """An error completion leaves the jetty in the ERROR state (new posts are refused): flush what is queued and
        return it to READY. Returns the number of flushed work requests."""
        n = self.lib.urma_simple_ep_recover(self.handle)
        if n < 0:
            raise UrmaError("cannot recover the endpoint")
        return n

    def _collect(self, fn, max_n):
        st = (ctypes.c_int * max_n)()
        uc = (ctypes.c_uint64 * max_n)()
        ln = (ctypes.c_uint32 * max_n)()
        im = (ctypes.c_uint64 * max_n)()
        fl = (ctypes.c_uint32 * max_n)()
        n = fn(self.handle, max_n, st, uc, ln, im, fl)
        return [Completion((st[i], uc[i], ln[i], im[i], fl[i])) for i in range(max(n, 0))]

    def close(self):
        if self.handle:
            self.lib.urma_simple_ep_destroy(self.handle)
            self.handle = None


class Context:
    def __init__(self, device: str = "shm0"):
        self.lib = _lib()
        self.handle = self.lib.urma_simple_open(device.encode())
        if not self.handle:
            raise UrmaError(f"cannot open URMA device {device!r}")
        self._children = []

    def endpoint(self, depth: int = 256, recv_token: int = 0, interrupt: bool = False) -> Endpoint:
        ep = Endpoint(self, depth, recv_token, interrupt)
        self._children.append(ep)
        return ep

    def register(self, buf, access: int = READ | WRITE | ATOMIC, token: int = 0) -> Segment:
        a, n = _addr_len(buf)
        blob = ctypes.create_string_buffer(SEG_BLOB)
        h = self.lib.urma_simple_seg_register(self.handle, a, n, access, token, blob)
        if not h:
            raise UrmaError("urma_register_seg failed (invalid access flags?)")
        s = Segment(self, h, bytes(blob.raw), False, keep=buf)
        self._children.append(s)
        return s

    def import_segment(self, blob: bytes, token: int = 0) -> Segment:
        h = self.lib.urma_simple_seg_import(self.handle, blob, token)
        if not h:
            raise UrmaError("urma_import_seg failed")
        s = Segment(self, h, blob, True)
        self._children.append(s)
        return s

    def import_endpoint(self, blob: bytes, token: int = 0) -> int:
        h = self.lib.urma_simple_ep_import(self.handle, blob, token)
        if not h:
            raise UrmaError("urma_import_jetty failed")
        self._children.append(("tj", h))
        return h

    def close(self):
        for c in reversed(self._children):
            if isinstance(c, tuple):
                self.lib.urma_unimport_jetty(c[1])
            else:
                c.close()
        self._children = []
        if self.handle:
            self.lib.urma_simple_close(self.handle)
            self.handle = None


class _CtlIn(ctypes.Structure):
    _fields_ = [("addr", ctypes.c_uint64), ("len", ctypes.c_uint32), ("opcode", ctypes.c_uint32)]


class _CtlOut(ctypes.Structure):
    _fields_ = [("addr", ctypes.c_uint64), ("len", ctypes.c_uint32), ("rsv", ctypes.c_uint32)]


def user_ctl(ctx: Context, opcode: int, addr: int = 0, length: int = 0, out_buf=None) -> int:
    """Provider-specific control call (urma_user_ctl). Returns the provider's 32-bit result word."""
    lib = _lib()
    lib.urma_user_ctl.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    cin = _CtlIn(addr, length, opcode)
    cout = _CtlOut(ctypes.addressof(out_buf) if out_buf is not None else 0,
                   ctypes.sizeof(out_buf) if out_buf is not None else 0, 0)
    rc = lib.urma_user_ctl(ctx.handle, ctypes.byref(cin), ctypes.byref(cout))
    if rc != 0:
        raise UrmaError(f"urma_user_ctl(opcode {opcode}) failed: {rc}")
    return cout.rsv


def bond_path_stats(ctx: Context):
    """[{up, tx, errors, failovers, failbacks, admin_down}] per physical path of a bond context."""
    buf = (ctypes.c_uint64 * (6 * 4))()
    n = user_ctl(ctx, 1, out_buf=buf)
    keys = ("up", "tx", "errors", "failovers", "failbacks", "admin_down")
    return [dict(zip(keys, [int(buf[i * 6 + k]) for k in range(6)])) for i in range(n)]


BOND_POLICIES = ("round_robin", "priority", "affinity", "least_load", "random")


def bond_set_policy(ctx: Context, policy: str, priority=None):
    """Path scheduling policy of a bond context in BALANCE mode (one of BOND_POLICIES); ``priority`` = path numbers,
    most preferred first (used by 'priority' and as the failover route of 'affinity')."""
    if priority is not None:
        packed = 0
        for k, p in enumerate(priority):
            packed |= (int(p) & 0xf) << (4 * k)
        user_ctl(ctx, 6, addr=packed)
    user_ctl(ctx, 5, addr=BOND_POLICIES.index(policy))


def bond_sched_stats(ctx: Context) -> dict:
    """{policy, deferred_resends, inflight: [per path]}: the scheduler's view of a bond context."""
    buf = (ctypes.c_uint64 * (2 + 4))()
    n = user_ctl(ctx, 7, out_buf=buf)
    return {"policy": BOND_POLICIES[int(buf[0])], "deferred_resends": int(buf[1]),
            "inflight": [int(buf[2 + i]) for i in range(n)]}

