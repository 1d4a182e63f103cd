"""Topology / aggregation-device registry (csrc/urma/uvs_topo.cpp) through its C API."""
import ctypes
import os

import pytest

from umdk_b200 import _native


class _In6(ctypes.Structure):
    _fields_ = [("hi", ctypes.c_uint64), ("lo", ctypes.c_uint64)]


class Eid(ctypes.Union):   # 8-byte aligned like the C union
    _fields_ = [("raw", ctypes.c_uint8 * 16), ("in6", _In6)]


class AggDev(ctypes.Structure):
    _fields_ = [("agg_eid", Eid), ("name", ctypes.c_char * 64), ("member_num", ctypes.c_uint32),
                ("member_eids", Eid * 8), ("member_names", (ctypes.c_char * 64) * 8)]


class Node(ctypes.Structure):
    _fields_ = [("type", ctypes.c_uint32), ("super_node_id", ctypes.c_uint32), ("node_id", ctypes.c_uint32),
                ("is_current", ctypes.c_uint32), ("port_num", ctypes.c_uint32), ("links", ctypes.c_uint64 * 18),
                ("primary_eid", Eid), ("port_eids", Eid * 18)]


class Path(ctypes.Structure):
    _fields_ = [("src_node", ctypes.c_uint32), ("dst_node", ctypes.c_uint32), ("src_port", ctypes.c_uint32),
                ("dst_port", ctypes.c_uint32), ("src_eid", Eid), ("dst_eid", Eid)]


class PathSet(ctypes.Structure):
    _fields_ = [("topo_type", ctypes.c_uint32), ("path_count", ctypes.c_uint32), ("paths", Path * 32)]


def _eid(tag: bytes, last: int) -> Eid:
    e = Eid()
    for i, b in enumerate(tag[:8]):
        e.raw[i] = b
    e.raw[15] = last
    return e


@pytest.fixture(scope="module")
def lib():
    path = os.path.join(_native.lib_dir(), "libumdk_urma.so")
    return ctypes.CDLL(path)


def test_agg_dev_registry(lib):
    agg = _eid(b"agg", 1)
    names = (ctypes.c_char_p * 2)(b"shm0", b"shm1")
    assert lib.uvs_create_agg_dev(ctypes.byref(agg), b"bondX", names, 2) == 0
    assert lib.uvs_create_agg_dev(ctypes.byref(agg), b"bondY", names, 2) < 0      # same EID
    out = AggDev()
    assert lib.uvs_get_agg_dev(b"bondX", ctypes.byref(out)) == 0
    assert out.member_num == 2 and out.member_names[1].value == b"shm1"
    buf = ctypes.create_string_buffer(64)
    assert lib.uvs_get_device_name_by_eid(ctypes.byref(agg), buf, 64) == 0 and buf.value == b"bondX"
    assert lib.uvs_delete_agg_dev(ctypes.byref(agg)) == 0
    assert lib.uvs_get_agg_dev(b"bondX", ctypes.byref(out)) < 0


def test_clos_planes_path_set_and_main_ue(lib):
    nodes = (Node * 3)()
    for i in range(3):
        n = nodes[i]
        n.type, n.node_id, n.is_current, n.port_num = 1, i, 1 if i == 0 else 0, 18
        n.primary_eid = _eid(b"gpu", i + 1)
        for p in range(18):
            n.links[p] = 0b111
            n.port_eids[p] = _eid(b"port%d" % i, p + 1)
    nodes[2].links[5] = 0          # node 2 lost plane 5
    assert lib.uvs_set_topo_info(nodes, 3) == 0
    cnt = ctypes.c_uint32()
    assert lib.uvs_get_topo_info(None, 0, ctypes.byref(cnt)) == 0 and cnt.value == 3
    ps = PathSet()
    assert lib.uvs_get_path_set(ctypes.byref(nodes[0].primary_eid), ctypes.byref(nodes[1].primary_eid), 0,
                                ctypes.byref(ps)) == 0
    assert ps.topo_type == 1 and ps.path_count == 18
    assert lib.uvs_get_path_set(ctypes.byref(nodes[0].primary_eid), ctypes.byref(nodes[2].primary_eid), 0,
                                ctypes.byref(ps)) == 0
    assert ps.path_count == 17 and all(ps.paths[i].src_port != 5 for i in range(17))
    # a virtual EID resolves through the main-UE table
    v = _eid(b"virt", 9)
    assert lib.uvs_get_path_set(ctypes.byref(v), ctypes.byref(nodes[1].primary_eid), 0, ctypes.byref(ps)) < 0
    assert lib.uvs_insert_main_ue_eid(ctypes.byref(v), ctypes.byref(nodes[0].primary_eid)) == 0
    assert lib.uvs_get_path_set(ctypes.byref(v), ctypes.byref(nodes[1].primary_eid), 0, ctypes.byref(ps)) == 0
    got = Eid()
    assert lib.uvs_lookup_main_ue_eid(ctypes.byref(v), ctypes.byref(got)) == 0 and bytes(got.raw) == bytes(
        nodes[0].primary_eid.raw)
    assert lib.uvs_flush_main_ue_eid() == 0
    assert lib.uvs_lookup_main_ue_eid(ctypes.byref(v), ctypes.byref(got)) < 0
    # two nodes marked current: refused
    nodes[1].is_current = 1
    assert lib.uvs_set_topo_info(nodes, 3) < 0


def test_discover_local_topology_lists_shm_devices(lib):
    from umdk_b200 import urma
    ctx = urma.Context("shm0")     # makes sure the library is initialised
    try:
        n = lib.uvs_discover_local_topology()
        assert n >= 1
        cnt = ctypes.c_uint32()
        assert lib.uvs_get_topo_info(None, 0, ctypes.byref(cnt)) == 0 and cnt.value == n
    finally:
        ctx.close()
