/* URMA (unified remote memory access) types: status codes, opcodes, completion records, object handles.
 * The names follow the reference's public API (src/urma/lib/urma/core/include/urma_types.h, urma_opcode.h) so that
 * code written against it keeps compiling; the layout and implementation are this project's own. Objects are
 * opaque to the application except for the documented fields. */
#ifndef UMDK_URMA_TYPES_H
#define UMDK_URMA_TYPES_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define URMA_EID_SIZE 16
#define URMA_MAX_NAME 64
#define URMA_MAX_SGE 8

typedef enum urma_status {
  URMA_SUCCESS = 0,
  URMA_EAGAIN = 11,
  URMA_ENOMEM = 12,
  URMA_ENOPERM = 13,
  URMA_ETIMEOUT = 110,
  URMA_EINVAL = 22,
  URMA_EEXIST = 17,
  URMA_EINPROGRESS = 115,
  URMA_FAIL = 0x1000,
} urma_status_t;

typedef enum urma_opcode {
  URMA_OPC_WRITE = 0x00,
  URMA_OPC_WRITE_IMM = 0x01,
  URMA_OPC_WRITE_NOTIFY = 0x02,
  URMA_OPC_READ = 0x10,
  URMA_OPC_CAS = 0x20,
  URMA_OPC_SWAP = 0x21,
  URMA_OPC_FADD = 0x22,
  URMA_OPC_FSUB = 0x23,
  URMA_OPC_FAND = 0x24,
  URMA_OPC_FOR = 0x25,
  URMA_OPC_FXOR = 0x26,
  URMA_OPC_SEND = 0x40,
  URMA_OPC_SEND_IMM = 0x41,
  URMA_OPC_SEND_INVALIDATE = 0x42,
  URMA_OPC_NOP = 0x51,
  URMA_OPC_LAST
} urma_opcode_t;

typedef enum urma_cr_status {
  URMA_CR_SUCCESS = 0,
  URMA_CR_UNSUPPORTED_OPCODE_ERR,
  URMA_CR_LOC_LEN_ERR,
  URMA_CR_LOC_OPERATION_ERR,
  URMA_CR_LOC_ACCESS_ERR,
  URMA_CR_REM_RESP_LEN_ERR,
  URMA_CR_REM_UNSUPPORTED_REQ_ERR,
  URMA_CR_REM_OPERATION_ERR,
  URMA_CR_REM_ACCESS_ABORT_ERR,
  URMA_CR_ACK_TIMEOUT_ERR,
  URMA_CR_RNR_RETRY_CNT_EXC_ERR,
  URMA_CR_WR_FLUSH_ERR,
  URMA_CR_WR_SUSPEND_DONE,
  URMA_CR_WR_FLUSH_ERR_DONE,
  URMA_CR_WR_UNHANDLED,
  URMA_CR_LOC_DATA_POISON,
  URMA_CR_REM_DATA_POISON
} urma_cr_status_t;

typedef enum urma_cr_opcode {
  URMA_CR_OPC_SEND = 0,
  URMA_CR_OPC_SEND_WITH_IMM,
  URMA_CR_OPC_SEND_WITH_INV,
  URMA_CR_OPC_WRITE_WITH_IMM
} urma_cr_opcode_t;

typedef enum urma_transport_mode { URMA_TM_RM = 1, URMA_TM_RC = 2, URMA_TM_UM = 4 } urma_transport_mode_t;
typedef enum urma_jetty_state {
  URMA_JETTY_STATE_RESET = 0,
  URMA_JETTY_STATE_READY,
  URMA_JETTY_STATE_SUSPENDED,
  URMA_JETTY_STATE_ERROR
} urma_jetty_state_t;
typedef enum urma_jfc_mode { URMA_JFC_POLLING = 0, URMA_JFC_INTERRUPT = 1 } urma_jfc_mode_t;

typedef enum urma_async_event_type {
  URMA_EVENT_JFC_ERR = 0,
  URMA_EVENT_JFS_ERR,
  URMA_EVENT_JFR_ERR,
  URMA_EVENT_JFR_LIMIT,
  URMA_EVENT_JETTY_ERR,
  URMA_EVENT_JETTY_LIMIT,
  URMA_EVENT_JETTY_GRP_ERR,
  URMA_EVENT_PORT_ACTIVE,
  URMA_EVENT_PORT_DOWN,
  URMA_EVENT_DEV_FATAL,
  URMA_EVENT_EID_CHANGE,
  URMA_EVENT_ELR_ERR,
  URMA_EVENT_ELR_DONE
} urma_async_event_type_t;

/* segment access bits (reference rules: LOCAL_ONLY is exclusive; WRITE needs READ; ATOMIC needs READ and WRITE) */
#define URMA_ACCESS_LOCAL_ONLY 0x1u
#define URMA_ACCESS_READ 0x2u
#define URMA_ACCESS_WRITE 0x4u
#define URMA_ACCESS_ATOMIC 0x8u

/* work-request flags */
#define URMA_WR_FLAG_COMPLETE_ENABLE 0x1u /* generate a completion record for this WR */
#define URMA_WR_FLAG_FENCE 0x2u
#define URMA_WR_FLAG_SOLICITED 0x4u
#define URMA_WR_FLAG_INLINE 0x8u

typedef union urma_eid {
  uint8_t raw[URMA_EID_SIZE];
  struct {
    uint64_t hi;
    uint64_t lo;
  } in6;
} urma_eid_t;

typedef struct urma_jetty_id {
  urma_eid_t eid;
  uint32_t uasid;
  uint32_t id;
} urma_jetty_id_t;

typedef struct urma_ubva {
  urma_eid_t eid;
  uint32_t uasid;
  uint64_t va;
} urma_ubva_t;

typedef struct urma_token {
  uint32_t token;
} urma_token_t;

typedef struct urma_seg {
  urma_ubva_t ubva;
  uint64_t len;
  uint32_t attr;     /* access bits */
  uint32_t token_id; /* index of the registration on the owner */
} urma_seg_t;

typedef struct urma_device_attr {
  uint32_t max_jfc, max_jfs, max_jfr, max_jetty, max_seg;
  uint32_t max_jfc_depth, max_jfs_depth, max_jfr_depth;
  uint32_t max_sge;
  uint64_t max_msg_size;
  uint32_t transport_modes; /* OR of urma_transport_mode_t */
  uint32_t port_cnt;
  bool atomic_supported;
} urma_device_attr_t;

typedef struct urma_device {
  char name[URMA_MAX_NAME];
  char provider[URMA_MAX_NAME];
  urma_eid_t eid;
  uint32_t index;
  void* priv; /* provider data */
} urma_device_t;

typedef struct urma_eid_info {
  urma_eid_t eid;
  uint32_t eid_index;
} urma_eid_info_t;

struct urma_ops;
typedef struct urma_context {
  urma_device_t* dev;
  const struct urma_ops* ops;
  urma_eid_t eid;
  uint32_t eid_index;
  uint32_t uasid;
  int async_fd;
  void* priv;
  volatile int refcnt;
} urma_context_t;

typedef struct urma_jfce {
  urma_context_t* ctx;
  int fd;
  void* priv;
} urma_jfce_t;

typedef struct urma_jfc_cfg {
  uint32_t depth;
  uint32_t flag;
  urma_jfce_t* jfce;
  uint64_t user_ctx;
} urma_jfc_cfg_t;

typedef struct urma_jfc {
  urma_context_t* ctx;
  urma_jfc_cfg_t cfg;
  uint32_t id;
  void* priv;
  volatile int refcnt;
} urma_jfc_t;

typedef struct urma_jfs_cfg {
  uint32_t depth;
  uint32_t flag;
  urma_transport_mode_t trans_mode;
  uint8_t priority;
  uint8_t max_sge;
  uint8_t rnr_retry;
  uint8_t err_timeout;
  urma_jfc_t* jfc;
  uint64_t user_ctx;
} urma_jfs_cfg_t;

typedef struct urma_jfs {
  urma_context_t* ctx;
  urma_jfs_cfg_t cfg;
  urma_jetty_id_t jfs_id;
  void* priv;
} urma_jfs_t;

typedef struct urma_jfr_cfg {
  uint32_t depth;
  uint32_t flag;
  urma_transport_mode_t trans_mode;
  uint8_t max_sge;
  uint8_t min_rnr_timer;
  urma_jfc_t* jfc;
  urma_token_t token_value;
  uint32_t id; /* 0 = let the provider choose */
  uint64_t user_ctx;
} urma_jfr_cfg_t;

typedef struct urma_jfr {
  urma_context_t* ctx;
  urma_jfr_cfg_t cfg;
  urma_jetty_id_t jfr_id;
  void* priv;
} urma_jfr_t;

typedef struct urma_jetty_grp urma_jetty_grp_t;

typedef struct urma_jetty_cfg {
  uint32_t id; /* 0 = let the provider choose */
  uint32_t flag;
  urma_jfs_cfg_t jfs_cfg;
  urma_jfr_cfg_t jfr_cfg; /* used when shared_jfr is NULL */
  urma_jfr_t* shared_jfr;
  urma_jetty_grp_t* jetty_grp;
  uint64_t user_ctx;
} urma_jetty_cfg_t;

typedef struct urma_target_jetty urma_target_jetty_t;

typedef struct urma_jetty {
  urma_context_t* ctx;
  urma_jetty_cfg_t cfg;
  urma_jetty_id_t jetty_id;
  urma_target_jetty_t* remote_jetty; /* set by bind (RC) */
  void* priv;
} urma_jetty_t;

typedef struct urma_rjetty {
  urma_jetty_id_t jetty_id;
  urma_transport_mode_t trans_mode;
  uint32_t type; /* 0 jfr, 1 jetty, 2 jetty group */
} urma_rjetty_t;
typedef urma_rjetty_t urma_rjfr_t;

struct urma_target_jetty {
  urma_context_t* ctx;
  urma_jetty_id_t id;
  urma_transport_mode_t trans_mode;
  uint32_t type;
  void* priv;
};

struct urma_jetty_grp {
  urma_context_t* ctx;
  urma_jetty_id_t id;
  char name[URMA_MAX_NAME];
  uint32_t policy; /* 0 round-robin, 1 hash */
  void* priv;
};

typedef struct urma_token_id {
  urma_context_t* ctx;
  uint32_t token_id;
} urma_token_id_t;

typedef struct urma_seg_cfg {
  uint64_t va;
  uint64_t len;
  urma_token_id_t* token_id; /* NULL = allocate one */
  urma_token_t token_value;
  uint32_t access;
  uint64_t user_ctx;
} urma_seg_cfg_t;

typedef struct urma_target_seg {
  urma_seg_t seg;
  urma_context_t* ctx;
  urma_token_id_t* token_id;
  uint64_t mva; /* locally mapped address when the provider maps remote memory (0 otherwise) */
  uint64_t user_ctx;
  bool is_import;
  bool own_token_id;
  void* priv;
} urma_target_seg_t;

typedef struct urma_sge {
  uint64_t addr;
  uint32_t len;
  urma_target_seg_t* tseg;
} urma_sge_t;

typedef struct urma_sg {
  urma_sge_t* sge;
  uint32_t num_sge;
} urma_sg_t;

typedef struct urma_rw_wr {
  urma_sg_t src;
  urma_sg_t dst;
  uint64_t notify_data; /* imm data for WRITE_IMM / value for WRITE_NOTIFY */
} urma_rw_wr_t;

typedef struct urma_send_wr {
  urma_sg_t src;
  uint64_t imm_data;
  urma_target_seg_t* tseg; /* SEND_INVALIDATE */
} urma_send_wr_t;

typedef struct urma_cas_wr {
  urma_sge_t* dst; /* remote 8-byte word */
  urma_sge_t* src; /* local buffer that receives the old value */
  uint64_t cmp_data;
  uint64_t swap_data;
} urma_cas_wr_t;

typedef struct urma_faa_wr {
  urma_sge_t* dst;
  urma_sge_t* src; /* local buffer that receives the old value */
  uint64_t operand;
} urma_faa_wr_t;

typedef struct urma_jfs_wr {
  urma_opcode_t opcode;
  uint32_t flag;
  urma_target_jetty_t* tjetty;
  uint64_t user_ctx;
  union {
    urma_rw_wr_t rw;
    urma_send_wr_t send;
    urma_cas_wr_t cas;
    urma_faa_wr_t faa;
  };
  struct urma_jfs_wr* next;
} urma_jfs_wr_t;

typedef struct urma_jfr_wr {
  urma_sg_t src; /* receive buffers */
  uint64_t user_ctx;
  struct urma_jfr_wr* next;
} urma_jfr_wr_t;

typedef struct urma_cr {
  urma_cr_status_t status;
  uint64_t user_ctx;
  urma_cr_opcode_t opcode;
  uint32_t flag; /* bit0: 1 = receive side, 0 = send side */
  uint32_t completion_len;
  uint32_t local_id;
  urma_jetty_id_t remote_id;
  uint64_t imm_data;
  uint32_t tpn;
  uintptr_t user_data;
} urma_cr_t;
#define URMA_CR_FLAG_RECV 0x1u

typedef struct urma_async_event {
  urma_context_t* ctx;
  urma_async_event_type_t event_type;
  union {
    urma_jfc_t* jfc;
    urma_jfs_t* jfs;
    urma_jfr_t* jfr;
    urma_jetty_t* jetty;
    uint32_t port_id;
  } element;
  void* priv;
} urma_async_event_t;

typedef struct urma_init_attr {
  uint64_t token;
  uint32_t uasid; /* 0 = assign */
  const char* provider_dir; /* extra directory scanned for liburma-*.so providers (may be NULL) */
} urma_init_attr_t;

typedef struct urma_user_ctl_in {
  uint64_t addr;
  uint32_t len;
  uint32_t opcode;
} urma_user_ctl_in_t;
typedef struct urma_user_ctl_out {
  uint64_t addr;
  uint32_t len;
  uint32_t rsv;
} urma_user_ctl_out_t;

typedef enum urma_vlog_level {
  URMA_VLOG_LEVEL_EMERG = 0,
  URMA_VLOG_LEVEL_ALERT,
  URMA_VLOG_LEVEL_CRIT,
  URMA_VLOG_LEVEL_ERR,
  URMA_VLOG_LEVEL_WARNING,
  URMA_VLOG_LEVEL_NOTICE,
  URMA_VLOG_LEVEL_INFO,
  URMA_VLOG_LEVEL_DEBUG
} urma_vlog_level_t;
typedef void (*urma_log_cb_t)(int level, char* message);
/* like urma_log_cb_t, with the source location as separate arguments */
typedef void (*urma_loc_log_cb)(int level, const char* function, int line, const char* message);

/* ---- extended control plane (urma_ext.cpp) ---- */
/* Options of urma_set_*_opt / urma_get_*_opt. "rw": may be changed between urma_alloc_* and urma_active_*;
 * "ro": fixed by the cfg given to urma_alloc_*, readable at any time. */
typedef enum urma_opt_name {
  URMA_OPT_DEPTH = 1,            /* ro uint32 */
  URMA_OPT_FLAG = 2,             /* ro uint32 */
  URMA_OPT_USER_CTX = 3,         /* rw uint64 */
  URMA_OPT_TRANS_MODE = 4,       /* ro uint32 (jfs, jfr, jetty) */
  URMA_OPT_PRIORITY = 5,         /* rw uint8 (jfs, jetty) */
  URMA_OPT_RNR_RETRY = 6,        /* rw uint8 (jfs, jetty) */
  URMA_OPT_ERR_TIMEOUT = 7,      /* rw uint8 (jfs, jetty) */
  URMA_OPT_MIN_RNR_TIMER = 8,    /* rw uint8 (jfr, jetty) */
  URMA_OPT_MODERATE_COUNT = 9,   /* rw uint32 (jfc): completions per event */
  URMA_OPT_MODERATE_PERIOD = 10, /* rw uint32 (jfc): microseconds */
  URMA_OPT_RX_THRESHOLD = 11,    /* rw uint32 (jfr): low-watermark event */
  URMA_OPT_ID = 12,              /* ro uint32: the object's id */
  URMA_OPT_STATE = 13,           /* ro uint32: urma_jetty_state_t (jfs, jfr, jetty); 1 when active (jfc) */
  URMA_OPT_CTX_LOG_TAG = 100,    /* rw string (context): tag put into this thread's log lines by context calls */
  URMA_OPT_CTX_USER_DATA = 101   /* rw uint64 (context) */
} urma_opt_name_t;

typedef enum urma_notify_type { URMA_IMPORT_JETTY_NOTIFY = 0, URMA_BIND_JETTY_NOTIFY = 1, URMA_ADVISE_JFR_NOTIFY = 2 }
    urma_notify_type_t;
typedef struct urma_notify {
  urma_notify_type_t type;
  urma_status_t status;
  uint64_t user_ctx;
  union {
    urma_target_jetty_t* tjetty; /* import, advise */
    urma_jetty_t* jetty;         /* bind */
  };
} urma_notify_t;
typedef struct urma_notifier {
  urma_context_t* ctx;
  int fd; /* readable while notifications are pending (eventfd) */
  void* priv;
} urma_notifier_t;
typedef void (*urma_advise_async_cb_func)(urma_status_t status, void* arg);

typedef struct urma_import_jetty_ex_cfg {
  uint64_t tp_handle;      /* 0 = let the library pick the transport path */
  uint64_t peer_tp_handle;
  uint64_t tag;
} urma_import_jetty_ex_cfg_t;
typedef urma_import_jetty_ex_cfg_t urma_import_jfr_ex_cfg_t;
typedef urma_import_jetty_ex_cfg_t urma_bind_jetty_ex_cfg_t;
typedef union urma_token_id_flag {
  struct {
    uint32_t multi_seg : 1; /* the id may cover several segments */
    uint32_t reserved : 31;
  } bs;
  uint32_t value;
} urma_token_id_flag_t;

/* transport paths and addressing */
#define URMA_IP_ADDR_BYTES 16
#define URMA_MAC_BYTES 6
typedef struct urma_net_addr {
  uint32_t sin_family; /* AF_INET or AF_INET6 */
  uint8_t addr[URMA_IP_ADDR_BYTES]; /* IPv4 in the first 4 bytes */
  uint16_t vlan;
  uint8_t mac[URMA_MAC_BYTES];
  uint32_t prefix_len;
} urma_net_addr_t;
typedef struct urma_net_addr_info {
  urma_net_addr_t netaddr;
  uint32_t index;
} urma_net_addr_info_t;
typedef struct urma_get_tp_cfg {
  uint32_t flag;
  urma_transport_mode_t trans_mode;
  urma_eid_t local_eid;
  urma_eid_t peer_eid;
} urma_get_tp_cfg_t;
typedef struct urma_tp_info {
  uint64_t tp_handle;
} urma_tp_info_t;
typedef struct urma_tp_attr_value {
  uint8_t retry_times_init;
  uint8_t at;
  uint8_t sip[URMA_IP_ADDR_BYTES];
  uint8_t dip[URMA_IP_ADDR_BYTES];
  uint8_t sma[URMA_MAC_BYTES];
  uint8_t dma[URMA_MAC_BYTES];
  uint16_t vlan_id;
  uint8_t vlan_en;
  uint8_t dscp;
  uint8_t at_times;
  uint8_t sl;
  uint8_t ttl;
  uint16_t ack_udp_srcport;
  uint16_t data_udp_srcport;
} urma_tp_attr_value_t;
/* bits of tp_attr_bitmap, in the order of the fields above */
enum { URMA_TP_ATTR_RETRY = 1u << 0, URMA_TP_ATTR_AT = 1u << 1, URMA_TP_ATTR_SIP = 1u << 2, URMA_TP_ATTR_DIP = 1u << 3,
       URMA_TP_ATTR_SMA = 1u << 4, URMA_TP_ATTR_DMA = 1u << 5, URMA_TP_ATTR_VLAN = 1u << 6, URMA_TP_ATTR_DSCP = 1u << 7,
       URMA_TP_ATTR_SL = 1u << 8, URMA_TP_ATTR_TTL = 1u << 9, URMA_TP_ATTR_UDP_PORTS = 1u << 10 };
typedef struct urma_tp_cfg {
  urma_transport_mode_t trans_mode;
  urma_eid_t local_eid;
  urma_eid_t peer_eid;
} urma_tp_cfg_t;
typedef struct urma_tp_attr {
  uint32_t peer_tpn;
  uint32_t state; /* 0 reset, 1 ready, 2 error */
  uint32_t tx_psn, rx_psn;
  uint32_t mtu;
} urma_tp_attr_t;
typedef uint32_t urma_tp_attr_mask_t; /* bit 0 peer_tpn, 1 state, 2 tx_psn, 3 rx_psn, 4 mtu */

#ifdef __cplusplus
}
#endif
#endif
