"""Secure control channel (TLS 1.3 with a pre-shared key) and message sealing (AES-256-GCM) of the host libraries."""
import ctypes
import os
import socket
import threading

import pytest

from umdk_b200 import _native

PSK = "00112233445566778899aabbccddeeff" * 2
OTHER = "ff" * 32


def _lib():
    lib = _native.urma()
    lib.ub_secure_seal.restype = ctypes.c_long
    lib.ub_secure_open.restype = ctypes.c_long
    lib.ub_secure_seal.argtypes = lib.ub_secure_open.argtypes = [
        ctypes.c_char_p, ctypes.c_char_p, ctypes.c_uint32, ctypes.c_uint64, ctypes.c_char_p, ctypes.c_size_t,
        ctypes.c_char_p, ctypes.c_size_t, ctypes.c_char_p, ctypes.c_size_t]
    lib.ub_secure_echo.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_char_p, ctypes.c_char_p, ctypes.c_size_t,
                                   ctypes.c_int, ctypes.c_char_p, ctypes.c_size_t]
    return lib


def _echo_pair(lib, psk_srv, psk_cli, id_srv=b"umdk", id_cli=b"umdk", n=100000):
    a, b = socket.socketpair()
    out = {}

    def srv():
        c = ctypes.create_string_buffer(64)
        out["srv"] = lib.ub_secure_echo(a.fileno(), 1, psk_srv, id_srv, n, 3000, c, 64)
        out["srv_cipher"] = c.value.decode()
    t = threading.Thread(target=srv)
    t.start()
    c = ctypes.create_string_buffer(64)
    out["cli"] = lib.ub_secure_echo(b.fileno(), 0, psk_cli, id_cli, n, 3000, c, 64)
    out["cli_cipher"] = c.value.decode()
    b.close()
    t.join()
    a.close()
    return out


def test_tls_psk_echo_negotiates_aes256_gcm():
    out = _echo_pair(_lib(), PSK.encode(), PSK.encode())
    assert out["srv"] == 0 and out["cli"] == 0
    assert out["cli_cipher"] == out["srv_cipher"] == "TLS_AES_256_GCM_SHA384"


def test_plain_passthrough_without_key():
    out = _echo_pair(_lib(), b"", b"")
    assert out["srv"] == 0 and out["cli"] == 0 and out["cli_cipher"] == "none"


@pytest.mark.parametrize("psk_cli,id_cli", [(OTHER.encode(), b"umdk"), (PSK.encode(), b"someone-else")])
def test_wrong_key_or_identity_fails_the_handshake(psk_cli, id_cli):
    out = _echo_pair(_lib(), PSK.encode(), psk_cli, id_cli=id_cli, n=64)
    assert out["srv"] == -3 and out["cli"] == -3


def test_clear_text_client_is_refused_by_a_secured_server():
    out = _echo_pair(_lib(), PSK.encode(), b"", n=64)
    assert out["srv"] != 0 and out["cli"] != 0


def test_seal_open_roundtrip_and_tamper_detection():
    lib = _lib()
    msg = os.urandom(1000)
    aad = b"header"
    sealed = ctypes.create_string_buffer(len(msg) + 16)
    n = lib.ub_secure_seal(PSK.encode(), b"dlock-cmd", 7, 42, aad, len(aad), msg, len(msg), sealed, len(sealed))
    assert n == len(msg) + 16 and sealed.raw[:len(msg)] != msg
    plain = ctypes.create_string_buffer(len(msg))
    assert lib.ub_secure_open(PSK.encode(), b"dlock-cmd", 7, 42, aad, len(aad), sealed.raw, n, plain, len(plain)) == len(msg)
    assert plain.raw == msg
    # wrong sequence number (replay under another nonce), wrong label (another derived key), changed header, flipped bit
    assert lib.ub_secure_open(PSK.encode(), b"dlock-cmd", 7, 43, aad, len(aad), sealed.raw, n, plain, len(plain)) == -1
    assert lib.ub_secure_open(PSK.encode(), b"urpc-data", 7, 42, aad, len(aad), sealed.raw, n, plain, len(plain)) == -1
    assert lib.ub_secure_open(PSK.encode(), b"dlock-cmd", 7, 42, b"headex", 6, sealed.raw, n, plain, len(plain)) == -1
    bad = bytearray(sealed.raw)
    bad[10] ^= 1
    assert lib.ub_secure_open(PSK.encode(), b"dlock-cmd", 7, 42, aad, len(aad), bytes(bad), n, plain, len(plain)) == -1
