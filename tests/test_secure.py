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


# ------------------------------------------------------------------------------------------------ certificates
def _make_pki(tmp_path, name):
    """A CA and two leaf certificates (server, client) signed by it, as PEM files."""
    import datetime
    from cryptography import x509
    from cryptography.hazmat.primitives import hashes, serialization
    from cryptography.hazmat.primitives.asymmetric import ec
    from cryptography.x509.oid import NameOID

    def write(path, data):
        path.write_bytes(data)
        return str(path)

    def key_pem(k):
        return k.private_bytes(serialization.Encoding.PEM, serialization.PrivateFormat.PKCS8,
                               serialization.NoEncryption())
    now = datetime.datetime.now(datetime.timezone.utc)
    ca_key = ec.generate_private_key(ec.SECP384R1())
    ca_name = x509.Name([x509.NameAttribute(NameOID.COMMON_NAME, f"{name} test CA")])
    ca = (x509.CertificateBuilder().subject_name(ca_name).issuer_name(ca_name).public_key(ca_key.public_key())
          .serial_number(x509.random_serial_number()).not_valid_before(now - datetime.timedelta(days=1))
          .not_valid_after(now + datetime.timedelta(days=30))
          .add_extension(x509.BasicConstraints(ca=True, path_length=None), critical=True)
          .sign(ca_key, hashes.SHA384()))
    out = {"ca": write(tmp_path / f"{name}_ca.pem", ca.public_bytes(serialization.Encoding.PEM))}
    for leaf in ("server", "client"):
        k = ec.generate_private_key(ec.SECP384R1())
        cert = (x509.CertificateBuilder()
                .subject_name(x509.Name([x509.NameAttribute(NameOID.COMMON_NAME, f"{name} {leaf}")]))
                .issuer_name(ca_name).public_key(k.public_key()).serial_number(x509.random_serial_number())
                .not_valid_before(now - datetime.timedelta(days=1)).not_valid_after(now + datetime.timedelta(days=30))
                .add_extension(x509.BasicConstraints(ca=False, path_length=None), critical=True)
                .sign(ca_key, hashes.SHA384()))
        out[leaf] = (write(tmp_path / f"{name}_{leaf}.pem", cert.public_bytes(serialization.Encoding.PEM)),
                     write(tmp_path / f"{name}_{leaf}.key", key_pem(k)))
    return out


def _echo_pair_cert(lib, srv_files, cli_files, n=50000):
    a, b = socket.socketpair()
    out = {}

    def server():
        c = ctypes.create_string_buffer(64)
        out["srv"] = lib.ub_secure_echo_cert(a.fileno(), 1, *[f.encode() for f in srv_files], n, 3000, c, 64)
        out["srv_cipher"] = c.value
    t = threading.Thread(target=server)
    t.start()
    c = ctypes.create_string_buffer(64)
    out["cli"] = lib.ub_secure_echo_cert(b.fileno(), 0, *[f.encode() for f in cli_files], n, 3000, c, 64)
    out["cli_cipher"] = c.value
    b.close()   # a refused client must not leave the server waiting for its timeout
    t.join()
    a.close()
    return out


def test_tls_with_certificates_mutual_authentication(tmp_path):
    lib = _lib()
    lib.ub_secure_echo_cert.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_char_p, ctypes.c_char_p, ctypes.c_char_p,
                                        ctypes.c_size_t, ctypes.c_int, ctypes.c_char_p, ctypes.c_size_t]
    ours, theirs = _make_pki(tmp_path, "ours"), _make_pki(tmp_path, "theirs")
    good = _echo_pair_cert(lib, (ours["ca"], *ours["server"]), (ours["ca"], *ours["client"]))
    assert good["srv"] == 0 and good["cli"] == 0
    assert good["cli_cipher"] == b"TLS_AES_256_GCM_SHA384" == good["srv_cipher"]
    # a client whose certificate comes from another CA is refused by the server ...
    bad = _echo_pair_cert(lib, (ours["ca"], *ours["server"]), (ours["ca"], *theirs["client"]), n=64)
    assert bad["srv"] != 0 and bad["cli"] != 0
    # ... and a client refuses a server that is not signed by the CA it trusts
    bad = _echo_pair_cert(lib, (theirs["ca"], *theirs["server"]), (ours["ca"], *ours["client"]), n=64)
    assert bad["cli"] != 0
    # a key that does not belong to the certificate never gets as far as a handshake
    bad = _echo_pair_cert(lib, (ours["ca"], *ours["server"]), (ours["ca"], ours["client"][0], ours["server"][1]), n=64)
    assert bad["cli"] != 0


def test_dlock_and_urpc_services_with_certificates(tmp_path):
    """The lock service and the RPC framework with certificate files instead of a shared key: peers of the same CA
    work (control channel in TLS 1.3, payloads sealed), a client with a certificate of another CA cannot join."""
    os.environ["URMA_SHM_DIR"] = str(tmp_path / "urma")
    (tmp_path / "urma").mkdir(exist_ok=True)
    from umdk_b200 import dlock, urpc
    ours, theirs = _make_pki(tmp_path, "ours"), _make_pki(tmp_path, "theirs")
    srv = None
    try:
        dlock.set_tls_files(ours["ca"], *ours["server"])
        srv = dlock.Server()                                  # keeps the files it was started with
        dlock.set_tls_files(ours["ca"], *ours["client"])
        a, b = dlock.Client(srv.ip, srv.port), dlock.Client(srv.ip, srv.port)
        la, lb = a.get_lock("C1", dlock.ATOMIC), b.get_lock("C1", dlock.ATOMIC)
        assert a.trylock(la) is True and b.trylock(lb) is False
        a.unlock(la)
        assert b.trylock(lb) is True
        b.unlock(lb)
        st = srv.stats()
        assert st["tls_rejected"] == 0 and st["sealed_rejected"] == 0 and st["data_msgs"] >= 3
        dlock.set_tls_files(ours["ca"], *theirs["client"])
        with pytest.raises(dlock.DlockError):
            dlock.Client(srv.ip, srv.port)
        dlock.set_tls_files()                                 # clear text against a server that wants certificates
        with pytest.raises(dlock.DlockError):
            dlock.Client(srv.ip, srv.port)
        assert srv.stats()["tls_rejected"] == 2
        with pytest.raises(dlock.DlockError):
            dlock.set_tls_files(ours["ca"], "", "")           # all three files or none
        a.close()
        b.close()
    finally:
        if srv is not None:
            srv.stop()
        dlock.set_psk("", "")

    urpc.init(default_timeout_ms=2000)
    rsrv = None
    try:
        urpc.set_tls_files(ours["ca"], *ours["server"])
        rsrv = urpc.Server()
        rsrv.register(1, lambda x: x[::-1])
        urpc.set_tls_files(ours["ca"], *ours["client"])
        ch = urpc.Channel(rsrv.ip, rsrv.port, queues=2)
        big = bytes(range(256)) * 100
        assert ch.call(1, b"with certificates") == b"setacifitrec htiw" and ch.call(1, big) == big[::-1]
        rep = urpc.admin_query("sessions")
        assert "TLS_AES_256_GCM_SHA384" in rep and "payload sealed" in rep
        ch.close()
        urpc.set_tls_files(ours["ca"], *theirs["client"])
        with pytest.raises(urpc.UrpcError):
            urpc.Channel(rsrv.ip, rsrv.port)
    finally:
        if rsrv is not None:
            rsrv.stop()
        urpc.set_psk("", "")
        urpc.uninit()
