// Secure control channels and message sealing for the host libraries.
//
// SecureConn wraps a connected TCP socket. With an empty pre-shared key it is a plain pass-through; with a key the
// two sides run a TLS 1.3 handshake in PSK mode restricted to TLS_AES_256_GCM_SHA384 and every later byte travels in
// TLS records. With certificate files instead of a key the handshake is TLS 1.3 with mutual authentication: each
// side presents its certificate and accepts only a peer whose chain ends at the configured CA. AeadCipher seals single messages (AES-256-GCM, 96-bit nonce = 32-bit salt || 64-bit sequence number)
// for data-plane traffic that does not go through the socket; its key is derived from the pre-shared key with
// HKDF-SHA256 and a per-use label.
//
// Same roles as the reference's control-channel security: URPC's TLS-PSK handshaker option
// (src/urpc/framework/lib/control/crypto/crypto.c), DLock's TLS 1.3 control connection and AES-GCM data-channel cipher
// (src/ulock/dlock/lib/common/ssl_connection.cpp, dlock_cipher.cpp) and the UMS agent's TLS token exchange
// (src/usock/ums/ums_agent/ums_agent_tls_conn.c).
#pragma once

#include <cstddef>
#include <cstdint>
#include <memory>
#include <string>
#include <vector>

#define UB_PUBLIC __attribute__((visibility("default")))

namespace ub {

struct UB_PUBLIC PskConfig {
  std::string identity = "umdk";
  std::vector<uint8_t> key;  // 16..64 bytes; empty = no pre-shared key
  // Certificate mode (takes precedence over the key): PEM files of the CA that signs the peers, of this side's
  // certificate chain and of its private key. All three or none.
  std::string ca_file, cert_file, key_file;

  bool use_certs() const { return !cert_file.empty(); }
  bool enabled() const { return !key.empty() || use_certs(); }
  // Reads <PREFIX>_PSK (hex string, 32..128 digits), <PREFIX>_PSK_ID and <PREFIX>_TLS_CA / _TLS_CERT / _TLS_KEY. A
  // malformed key or an incomplete set of files leaves the config disabled and sets *bad (when given) so that callers
  // can refuse to start instead of silently running in the clear.
  static PskConfig from_env(const char* prefix, bool* bad = nullptr);
  static bool parse_hex(const char* hex, std::vector<uint8_t>* out);
};

class UB_PUBLIC SecureConn {
 public:
  ~SecureConn();
  SecureConn(const SecureConn&) = delete;
  SecureConn& operator=(const SecureConn&) = delete;

  // Take a connected socket (not owned: the caller closes the fd after destroying the object). Return null and fill
  // *err when the handshake fails or times out.
  static std::unique_ptr<SecureConn> client(int fd, const PskConfig& cfg, int timeout_ms, std::string* err = nullptr);
  static std::unique_ptr<SecureConn> server(int fd, const PskConfig& cfg, int timeout_ms, std::string* err = nullptr);

  bool read_full(void* buf, size_t n, int timeout_ms);
  bool write_full(const void* buf, size_t n);
  bool pending() const;       // decrypted bytes already buffered (a poll() on the fd would not report them)
  bool encrypted() const { return ssl_ != nullptr; }
  const char* cipher() const;  // "none" or the negotiated suite
  int fd() const { return fd_; }

 private:
  SecureConn() = default;
  static std::unique_ptr<SecureConn> make(int fd, const PskConfig& cfg, bool is_server, int timeout_ms,
                                          std::string* err);
  int fd_ = -1;
  void* ctx_ = nullptr;  // SSL_CTX
  void* ssl_ = nullptr;  // SSL
  PskConfig cfg_;
  friend struct SecureConnCallbacks;
};

// out = HKDF-SHA256(key = cfg.key, salt = salt bytes, info = label). False when security is off.
UB_PUBLIC bool derive_key(const PskConfig& cfg, const char* label, const void* salt, size_t salt_len, uint8_t out[32]);

class UB_PUBLIC AeadCipher {
 public:
  static constexpr size_t kTagBytes = 16;
  AeadCipher(const uint8_t key[32], uint32_t salt);
  ~AeadCipher();
  AeadCipher(const AeadCipher&) = delete;
  AeadCipher& operator=(const AeadCipher&) = delete;
  // out must hold n + kTagBytes bytes. aad is authenticated but not encrypted (may be null).
  bool seal(uint64_t seq, const void* aad, size_t aad_len, const void* in, size_t n, uint8_t* out);
  // in holds n_sealed = plaintext length + kTagBytes bytes; false on a bad tag (out is then unspecified).
  bool open(uint64_t seq, const void* aad, size_t aad_len, const uint8_t* in, size_t n_sealed, void* out);

 private:
  uint8_t key_[32];
  uint32_t salt_;
  void* ectx_ = nullptr;  // EVP_CIPHER_CTX, sealing
  void* dctx_ = nullptr;  // EVP_CIPHER_CTX, opening
};

UB_PUBLIC bool random_bytes(void* out, size_t n);

}  // namespace ub

// C entry points (for bindings and tests)
extern "C" {
// Seals / opens one message with a key derived from (psk_hex, label). Returns the output length or -1.
long ub_secure_seal(const char* psk_hex, const char* label, uint32_t salt, uint64_t seq, const void* aad, size_t aad_len,
                    const void* in, size_t n, void* out, size_t out_cap);
long ub_secure_open(const char* psk_hex, const char* label, uint32_t salt, uint64_t seq, const void* aad, size_t aad_len,
                    const void* in, size_t n, void* out, size_t out_cap);
// Runs one side of an echo over a SecureConn on an already connected socket: the client sends `n` bytes and checks
// the echo, the server echoes once. Returns 0 on success, a negative number on handshake / IO failure; when `cipher`
// is given the negotiated suite name is copied there.
int ub_secure_echo(int fd, int is_server, const char* psk_hex, const char* identity, size_t n, int timeout_ms,
                   char* cipher, size_t cipher_cap);
// The same over a certificate-authenticated connection.
int ub_secure_echo_cert(int fd, int is_server, const char* ca_file, const char* cert_file, const char* key_file, size_t n,
                        int timeout_ms, char* cipher, size_t cipher_cap);
}
