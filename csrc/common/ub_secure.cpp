#include "ub_secure.h"

#include <openssl/err.h>
#include <openssl/evp.h>
#include <openssl/kdf.h>
#include <openssl/rand.h>
#include <openssl/ssl.h>
#include <poll.h>
#include <sys/socket.h>
#include <sys/time.h>
#include <unistd.h>

#include <cstdlib>
#include <cstring>

namespace ub {

namespace {

// TLS 1.3 suite id of TLS_AES_256_GCM_SHA384
const unsigned char kSuiteId[2] = {0x13, 0x02};

void set_io_timeout(int fd, int ms) {
  timeval tv{ms / 1000, (ms % 1000) * 1000};
  setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
  setsockopt(fd, SOL_SOCKET, SO_SNDTIMEO, &tv, sizeof(tv));
}

std::string ssl_error_text(const char* what) {
  char buf[256];
  const unsigned long e = ERR_get_error();
  if (e) {
    ERR_error_string_n(e, buf, sizeof(buf));
  } else {
    snprintf(buf, sizeof(buf), "no detail (peer closed, wrong key or timeout)");
  }
  ERR_clear_error();
  return std::string(what) + ": " + buf;
}

SSL_SESSION* make_psk_session(SSL* ssl, const PskConfig& cfg) {
  const SSL_CIPHER* cipher = SSL_CIPHER_find(ssl, kSuiteId);
  if (!cipher) return nullptr;
  SSL_SESSION* s = SSL_SESSION_new();
  if (!s) return nullptr;
  if (!SSL_SESSION_set1_master_key(s, cfg.key.data(), cfg.key.size()) || !SSL_SESSION_set_cipher(s, cipher) ||
      !SSL_SESSION_set_protocol_version(s, TLS1_3_VERSION)) {
    SSL_SESSION_free(s);
    return nullptr;
  }
  return s;
}

}  // namespace

struct SecureConnCallbacks {
  static int use_session(SSL* ssl, const EVP_MD* md, const unsigned char** id, size_t* idlen, SSL_SESSION** sess) {
    auto* self = static_cast<SecureConn*>(SSL_get_app_data(ssl));
    *id = nullptr;
    *idlen = 0;
    *sess = nullptr;
    if (!self) return 0;
    const SSL_CIPHER* cipher = SSL_CIPHER_find(ssl, kSuiteId);
    if (!cipher) return 0;
    // after a HelloRetryRequest the digest is fixed: offer the key only if it matches the suite's digest
    if (md && SSL_CIPHER_get_handshake_digest(cipher) != md) return 1;
    SSL_SESSION* s = make_psk_session(ssl, self->cfg_);
    if (!s) return 0;
    *sess = s;
    *id = reinterpret_cast<const unsigned char*>(self->cfg_.identity.data());
    *idlen = self->cfg_.identity.size();
    return 1;
  }
  static int find_session(SSL* ssl, const unsigned char* identity, size_t identity_len, SSL_SESSION** sess) {
    auto* self = static_cast<SecureConn*>(SSL_get_app_data(ssl));
    *sess = nullptr;
    if (!self) return 0;
    if (identity_len != self->cfg_.identity.size() ||
        memcmp(identity, self->cfg_.identity.data(), identity_len) != 0)
      return 1;  // unknown identity: go on without a key, which ends the handshake (there is no certificate)
    SSL_SESSION* s = make_psk_session(ssl, self->cfg_);
    if (!s) return 0;
    *sess = s;
    return 1;
  }
};

PskConfig PskConfig::from_env(const char* prefix, bool* bad) {
  PskConfig c;
  if (bad) *bad = false;
  const std::string p(prefix);
  if (const char* id = getenv((p + "_PSK_ID").c_str()))
    if (*id) c.identity = id;
  const char* hex = getenv((p + "_PSK").c_str());
  if (hex && *hex) {
    if (!parse_hex(hex, &c.key) || c.key.size() < 16 || c.key.size() > 64) {
      c.key.clear();
      if (bad) *bad = true;
    }
  }
  const char* ca = getenv((p + "_TLS_CA").c_str());
  const char* cert = getenv((p + "_TLS_CERT").c_str());
  const char* pkey = getenv((p + "_TLS_KEY").c_str());
  const int given = (ca && *ca ? 1 : 0) + (cert && *cert ? 1 : 0) + (pkey && *pkey ? 1 : 0);
  if (given == 3) {
    c.ca_file = ca;
    c.cert_file = cert;
    c.key_file = pkey;
  } else if (given != 0 && bad) {
    *bad = true;
  }
  return c;
}

bool PskConfig::parse_hex(const char* hex, std::vector<uint8_t>* out) {
  out->clear();
  const size_t n = strlen(hex);
  if (n % 2) return false;
  auto nib = [](char ch) -> int {
    if (ch >= '0' && ch <= '9') return ch - '0';
    if (ch >= 'a' && ch <= 'f') return ch - 'a' + 10;
    if (ch >= 'A' && ch <= 'F') return ch - 'A' + 10;
    return -1;
  };
  for (size_t i = 0; i < n; i += 2) {
    const int hi = nib(hex[i]), lo = nib(hex[i + 1]);
    if (hi < 0 || lo < 0) {
      out->clear();
      return false;
    }
    out->push_back(static_cast<uint8_t>(hi * 16 + lo));
  }
  return true;
}

SecureConn::~SecureConn() {
  if (ssl_) {
    SSL* ssl = static_cast<SSL*>(ssl_);
    set_io_timeout(fd_, 200);
    SSL_shutdown(ssl);  // best effort close_notify; the peer may be gone already
    SSL_free(ssl);
  }
  if (ctx_) SSL_CTX_free(static_cast<SSL_CTX*>(ctx_));
}

std::unique_ptr<SecureConn> SecureConn::make(int fd, const PskConfig& cfg, bool is_server, int timeout_ms,
                                             std::string* err) {
  std::unique_ptr<SecureConn> c(new SecureConn());
  c->fd_ = fd;
  c->cfg_ = cfg;
  if (!cfg.enabled()) return c;
  SSL_CTX* ctx = SSL_CTX_new(is_server ? TLS_server_method() : TLS_client_method());
  if (!ctx) {
    if (err) *err = ssl_error_text("SSL_CTX_new");
    return nullptr;
  }
  c->ctx_ = ctx;
  SSL_CTX_set_min_proto_version(ctx, TLS1_3_VERSION);
  SSL_CTX_set_max_proto_version(ctx, TLS1_3_VERSION);
  SSL_CTX_set_ciphersuites(ctx, "TLS_AES_256_GCM_SHA384");
  SSL_CTX_set_mode(ctx, SSL_MODE_AUTO_RETRY);
  if (is_server) SSL_CTX_set_num_tickets(ctx, 0);  // no post-handshake messages: the first record after the handshake is data
  if (cfg.use_certs()) {
    // mutual authentication: present our chain, accept only a peer that presents one ending at the configured CA
    if (SSL_CTX_use_certificate_chain_file(ctx, cfg.cert_file.c_str()) != 1 ||
        SSL_CTX_use_PrivateKey_file(ctx, cfg.key_file.c_str(), SSL_FILETYPE_PEM) != 1 ||
        SSL_CTX_check_private_key(ctx) != 1 || SSL_CTX_load_verify_locations(ctx, cfg.ca_file.c_str(), nullptr) != 1) {
      if (err) *err = ssl_error_text("loading the certificate, key or CA file");
      return nullptr;
    }
    SSL_CTX_set_verify(ctx, SSL_VERIFY_PEER | SSL_VERIFY_FAIL_IF_NO_PEER_CERT, nullptr);
  } else if (is_server) {
    SSL_CTX_set_psk_find_session_callback(ctx, &SecureConnCallbacks::find_session);
  } else {
    SSL_CTX_set_psk_use_session_callback(ctx, &SecureConnCallbacks::use_session);
  }
  SSL* ssl = SSL_new(ctx);
  if (!ssl) {
    if (err) *err = ssl_error_text("SSL_new");
    return nullptr;
  }
  c->ssl_ = ssl;
  SSL_set_app_data(ssl, c.get());
  SSL_set_fd(ssl, fd);
  set_io_timeout(fd, timeout_ms > 0 ? timeout_ms : 5000);
  const int rc = is_server ? SSL_accept(ssl) : SSL_connect(ssl);
  if (rc != 1) {
    if (err) *err = ssl_error_text(is_server ? "TLS accept" : "TLS connect");
    return nullptr;
  }
  if (cfg.use_certs()) {
    X509* peer = SSL_get1_peer_certificate(ssl);
    const bool verified = peer && SSL_get_verify_result(ssl) == X509_V_OK;
    if (peer) X509_free(peer);
    if (!verified) {
      if (err) *err = "TLS handshake finished without a verified peer certificate";
      return nullptr;
    }
  } else if (!SSL_session_reused(ssl)) {  // a handshake that did not use the key cannot happen without certificates; be sure
    if (err) *err = "TLS handshake finished without the pre-shared key";
    return nullptr;
  }
  set_io_timeout(fd, 30000);  // safety net for a peer that stops in the middle of a record
  return c;
}

std::unique_ptr<SecureConn> SecureConn::client(int fd, const PskConfig& cfg, int timeout_ms, std::string* err) {
  return make(fd, cfg, false, timeout_ms, err);
}
std::unique_ptr<SecureConn> SecureConn::server(int fd, const PskConfig& cfg, int timeout_ms, std::string* err) {
  return make(fd, cfg, true, timeout_ms, err);
}

bool SecureConn::pending() const { return ssl_ && SSL_pending(static_cast<SSL*>(ssl_)) > 0; }

const char* SecureConn::cipher() const { return ssl_ ? SSL_get_cipher_name(static_cast<SSL*>(ssl_)) : "none"; }

bool SecureConn::read_full(void* buf, size_t n, int timeout_ms) {
  uint8_t* p = static_cast<uint8_t*>(buf);
  while (n) {
    if (!pending()) {
      pollfd pf{fd_, POLLIN, 0};
      if (poll(&pf, 1, timeout_ms) <= 0) return false;
    }
    ssize_t r;
    if (ssl_) {
      r = SSL_read(static_cast<SSL*>(ssl_), p, static_cast<int>(n > (1u << 30) ? (1u << 30) : n));
      if (r <= 0) {
        ERR_clear_error();
        return false;
      }
    } else {
      r = ::read(fd_, p, n);
      if (r <= 0) return false;
    }
    p += r;
    n -= static_cast<size_t>(r);
  }
  return true;
}

bool SecureConn::write_full(const void* buf, size_t n) {
  const uint8_t* p = static_cast<const uint8_t*>(buf);
  while (n) {
    ssize_t r;
    if (ssl_) {
      r = SSL_write(static_cast<SSL*>(ssl_), p, static_cast<int>(n > (1u << 30) ? (1u << 30) : n));
      if (r <= 0) {
        ERR_clear_error();
        return false;
      }
    } else {
      r = ::send(fd_, p, n, MSG_NOSIGNAL);
      if (r <= 0) return false;
    }
    p += r;
    n -= static_cast<size_t>(r);
  }
  return true;
}

bool derive_key(const PskConfig& cfg, const char* label, const void* salt, size_t salt_len, uint8_t out[32]) {
  if (!cfg.enabled()) return false;
  EVP_PKEY_CTX* pctx = EVP_PKEY_CTX_new_id(EVP_PKEY_HKDF, nullptr);
  if (!pctx) return false;
  size_t outlen = 32;
  const bool ok = EVP_PKEY_derive_init(pctx) > 0 && EVP_PKEY_CTX_set_hkdf_md(pctx, EVP_sha256()) > 0 &&
                  EVP_PKEY_CTX_set1_hkdf_salt(pctx, static_cast<const unsigned char*>(salt), (int)salt_len) > 0 &&
                  EVP_PKEY_CTX_set1_hkdf_key(pctx, cfg.key.data(), (int)cfg.key.size()) > 0 &&
                  EVP_PKEY_CTX_add1_hkdf_info(pctx, reinterpret_cast<const unsigned char*>(label),
                                              (int)strlen(label)) > 0 &&
                  EVP_PKEY_derive(pctx, out, &outlen) > 0 && outlen == 32;
  EVP_PKEY_CTX_free(pctx);
  return ok;
}

bool random_bytes(void* out, size_t n) { return RAND_bytes(static_cast<unsigned char*>(out), (int)n) == 1; }

AeadCipher::AeadCipher(const uint8_t key[32], uint32_t salt) : salt_(salt) {
  memcpy(key_, key, 32);
  ectx_ = EVP_CIPHER_CTX_new();
  dctx_ = EVP_CIPHER_CTX_new();
}

AeadCipher::~AeadCipher() {
  if (ectx_) EVP_CIPHER_CTX_free(static_cast<EVP_CIPHER_CTX*>(ectx_));
  if (dctx_) EVP_CIPHER_CTX_free(static_cast<EVP_CIPHER_CTX*>(dctx_));
  OPENSSL_cleanse(key_, sizeof(key_));
}

static void make_nonce(uint32_t salt, uint64_t seq, uint8_t nonce[12]) {
  memcpy(nonce, &salt, 4);
  memcpy(nonce + 4, &seq, 8);
}

bool AeadCipher::seal(uint64_t seq, const void* aad, size_t aad_len, const void* in, size_t n, uint8_t* out) {
  EVP_CIPHER_CTX* c = static_cast<EVP_CIPHER_CTX*>(ectx_);
  uint8_t nonce[12];
  make_nonce(salt_, seq, nonce);
  int len = 0, fin = 0;
  if (!c || EVP_EncryptInit_ex(c, EVP_aes_256_gcm(), nullptr, key_, nonce) != 1) return false;
  if (aad_len && EVP_EncryptUpdate(c, nullptr, &len, static_cast<const unsigned char*>(aad), (int)aad_len) != 1)
    return false;
  if (n && EVP_EncryptUpdate(c, out, &len, static_cast<const unsigned char*>(in), (int)n) != 1) return false;
  if (EVP_EncryptFinal_ex(c, out + n, &fin) != 1) return false;
  return EVP_CIPHER_CTX_ctrl(c, EVP_CTRL_GCM_GET_TAG, (int)kTagBytes, out + n) == 1;
}

bool AeadCipher::open(uint64_t seq, const void* aad, size_t aad_len, const uint8_t* in, size_t n_sealed, void* out) {
  if (n_sealed < kTagBytes) return false;
  const size_t n = n_sealed - kTagBytes;
  EVP_CIPHER_CTX* c = static_cast<EVP_CIPHER_CTX*>(dctx_);
  uint8_t nonce[12];
  make_nonce(salt_, seq, nonce);
  int len = 0, fin = 0;
  if (!c || EVP_DecryptInit_ex(c, EVP_aes_256_gcm(), nullptr, key_, nonce) != 1) return false;
  if (aad_len && EVP_DecryptUpdate(c, nullptr, &len, static_cast<const unsigned char*>(aad), (int)aad_len) != 1)
    return false;
  if (n && EVP_DecryptUpdate(c, static_cast<unsigned char*>(out), &len, in, (int)n) != 1) return false;
  if (EVP_CIPHER_CTX_ctrl(c, EVP_CTRL_GCM_SET_TAG, (int)kTagBytes, const_cast<uint8_t*>(in + n)) != 1) return false;
  return EVP_DecryptFinal_ex(c, static_cast<unsigned char*>(out) + n, &fin) == 1;
}

}  // namespace ub

#define UB_SECURE_EXPORT extern "C" __attribute__((visibility("default")))

static bool cipher_from(const char* psk_hex, const char* label, uint8_t key[32]) {
  ub::PskConfig cfg;
  if (!psk_hex || !ub::PskConfig::parse_hex(psk_hex, &cfg.key) || cfg.key.size() < 16) return false;
  return ub::derive_key(cfg, label ? label : "", "ub-secure", 9, key);
}

UB_SECURE_EXPORT long ub_secure_seal(const char* psk_hex, const char* label, uint32_t salt, uint64_t seq,
                                     const void* aad, size_t aad_len, const void* in, size_t n, void* out,
                                     size_t out_cap) {
  uint8_t key[32];
  if (out_cap < n + ub::AeadCipher::kTagBytes || !cipher_from(psk_hex, label, key)) return -1;
  ub::AeadCipher c(key, salt);
  return c.seal(seq, aad, aad_len, in, n, static_cast<uint8_t*>(out)) ? (long)(n + ub::AeadCipher::kTagBytes) : -1;
}

UB_SECURE_EXPORT long ub_secure_open(const char* psk_hex, const char* label, uint32_t salt, uint64_t seq,
                                     const void* aad, size_t aad_len, const void* in, size_t n, void* out,
                                     size_t out_cap) {
  uint8_t key[32];
  if (n < ub::AeadCipher::kTagBytes || out_cap < n - ub::AeadCipher::kTagBytes || !cipher_from(psk_hex, label, key))
    return -1;
  ub::AeadCipher c(key, salt);
  return c.open(seq, aad, aad_len, static_cast<const uint8_t*>(in), n, out) ? (long)(n - ub::AeadCipher::kTagBytes)
                                                                             : -1;
}

static int echo_over(int fd, int is_server, const ub::PskConfig& cfg, size_t n, int timeout_ms, char* cipher,
                     size_t cipher_cap);
UB_SECURE_EXPORT int ub_secure_echo(int fd, int is_server, const char* psk_hex, const char* identity, size_t n,
                                    int timeout_ms, char* cipher, size_t cipher_cap) {
  ub::PskConfig cfg;
  if (psk_hex && *psk_hex && !ub::PskConfig::parse_hex(psk_hex, &cfg.key)) return -2;
  if (identity && *identity) cfg.identity = identity;
  return echo_over(fd, is_server, cfg, n, timeout_ms, cipher, cipher_cap);
}
UB_SECURE_EXPORT int ub_secure_echo_cert(int fd, int is_server, const char* ca_file, const char* cert_file,
                                         const char* key_file, size_t n, int timeout_ms, char* cipher,
                                         size_t cipher_cap) {
  if (!ca_file || !cert_file || !key_file) return -2;
  ub::PskConfig cfg;
  cfg.ca_file = ca_file;
  cfg.cert_file = cert_file;
  cfg.key_file = key_file;
  return echo_over(fd, is_server, cfg, n, timeout_ms, cipher, cipher_cap);
}
static int echo_over(int fd, int is_server, const ub::PskConfig& cfg, size_t n, int timeout_ms, char* cipher,
                     size_t cipher_cap) {
  std::string err;
  auto conn = is_server ? ub::SecureConn::server(fd, cfg, timeout_ms, &err) : ub::SecureConn::client(fd, cfg, timeout_ms, &err);
  if (!conn) return -3;
  if (cipher && cipher_cap) snprintf(cipher, cipher_cap, "%s", conn->cipher());
  std::vector<uint8_t> buf(n), back(n);
  if (is_server) {
    if (!conn->read_full(buf.data(), n, timeout_ms) || !conn->write_full(buf.data(), n)) return -4;
    return 0;
  }
  for (size_t i = 0; i < n; ++i) buf[i] = static_cast<uint8_t>(i * 131 + 7);
  if (!conn->write_full(buf.data(), n) || !conn->read_full(back.data(), n, timeout_ms)) return -4;
  return memcmp(buf.data(), back.data(), n) == 0 ? 0 : -5;
}
