/* Flat convenience layer over the URMA API: one call creates a complete endpoint (event channel, completion queue,
 * jetty), descriptors of segments and jetties are plain byte blobs that can be sent over any out-of-band channel,
 * and every data-plane verb is one function taking integers. It carries the language bindings and the sample /
 * perftest tools; it follows the canonical sequence of the reference's sample program
 * (src/urma/examples/urma_sample.c:179-313: device -> context -> jfce/jfc/jfr/jetty -> register_seg -> exchange ->
 * import_seg/import_jetty -> write/read/send/recv -> poll). */
#ifndef UMDK_URMA_SIMPLE_H
#define UMDK_URMA_SIMPLE_H
#include "urma_api.h"
#ifdef __cplusplus
extern "C" {
#endif

#define URMA_SIMPLE_SEG_BLOB 64
#define URMA_SIMPLE_JETTY_BLOB 32

typedef struct urma_simple_ep urma_simple_ep_t;

URMA_EXPORT urma_context_t* urma_simple_open(const char* dev_name); /* runs urma_init on first use */
URMA_EXPORT int urma_simple_close(urma_context_t* ctx);
URMA_EXPORT urma_simple_ep_t* urma_simple_ep_create(urma_context_t* ctx, uint32_t depth, uint32_t recv_token,
                                                    int interrupt_mode);
URMA_EXPORT int urma_simple_ep_destroy(urma_simple_ep_t* ep);
URMA_EXPORT void urma_simple_ep_blob(urma_simple_ep_t* ep, uint8_t out[URMA_SIMPLE_JETTY_BLOB]);
URMA_EXPORT urma_target_jetty_t* urma_simple_ep_import(urma_context_t* ctx, const uint8_t blob[URMA_SIMPLE_JETTY_BLOB],
                                                       uint32_t token);
URMA_EXPORT urma_jetty_t* urma_simple_ep_jetty(urma_simple_ep_t* ep);
/* After an error completion the jetty is in the ERROR state and refuses new work requests: drain what is left and
 * put it back to READY. Returns the number of flushed work requests or < 0. */
URMA_EXPORT int urma_simple_ep_recover(urma_simple_ep_t* ep);
URMA_EXPORT urma_jfc_t* urma_simple_ep_jfc(urma_simple_ep_t* ep);

URMA_EXPORT urma_target_seg_t* urma_simple_seg_register(urma_context_t* ctx, void* va, uint64_t len, uint32_t access,
                                                        uint32_t token, uint8_t blob_out[URMA_SIMPLE_SEG_BLOB]);
URMA_EXPORT urma_target_seg_t* urma_simple_seg_import(urma_context_t* ctx, const uint8_t blob[URMA_SIMPLE_SEG_BLOB],
                                                      uint32_t token);

/* opcode: URMA_OPC_WRITE / READ / SEND / SEND_IMM / WRITE_IMM. rseg may be NULL for sends. */
URMA_EXPORT int urma_simple_post(urma_simple_ep_t* ep, urma_target_jetty_t* peer, int opcode,
                                 urma_target_seg_t* rseg, uint64_t raddr, urma_target_seg_t* lseg, uint64_t laddr,
                                 uint32_t len, uint64_t imm, uint64_t user_ctx, int signaled);
/* opcode: URMA_OPC_CAS / SWAP / FADD / FSUB / FAND / FOR / FXOR; old value is stored at *result (may be NULL). */
URMA_EXPORT int urma_simple_atomic(urma_simple_ep_t* ep, urma_target_jetty_t* peer, int opcode,
                                   urma_target_seg_t* rseg, uint64_t raddr, uint64_t operand, uint64_t compare,
                                   uint64_t* result, uint64_t user_ctx);
URMA_EXPORT int urma_simple_post_recv(urma_simple_ep_t* ep, void* buf, uint32_t len, uint64_t user_ctx);
/* Polls up to max completions; for each: status, user_ctx, len, imm, flag. Returns the count (or < 0). */
URMA_EXPORT int urma_simple_poll(urma_simple_ep_t* ep, int max, int* status, uint64_t* user_ctx, uint32_t* len,
                                 uint64_t* imm, uint32_t* flag);
/* Blocks until at least `want` completions arrived or timeout_ms elapsed; same outputs as poll. */
URMA_EXPORT int urma_simple_wait(urma_simple_ep_t* ep, int want, int timeout_ms, int max, int* status,
                                 uint64_t* user_ctx, uint32_t* len, uint64_t* imm, uint32_t* flag);
#ifdef __cplusplus
}
#endif
#endif
