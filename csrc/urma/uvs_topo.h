/*
 * Topology and aggregation-device registry (control-plane helper library).
 *
 * Role of the reference's UVS/TPSA library (src/urma/lib/uvs/core/include/uvs_api.h:146-207: aggregation devices,
 * topology set/get, main-UE EID table, path-set query), which there talks to the ubagg/uvs kernel modules by ioctl.
 * Here the registry lives in the process: it describes a box of GPUs behind NVSwitch planes (a Clos with parallel
 * planes: every port of every node reaches every other node through its own plane) or a full mesh of host devices,
 * and the bond provider asks it which physical devices make up an aggregation device and which port pairs connect
 * two of them.
 */
#ifndef UMDK_UVS_TOPO_H
#define UMDK_UVS_TOPO_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#include "urma_types.h"

#ifndef URMA_EXPORT
#define URMA_EXPORT __attribute__((visibility("default")))
#endif

#ifdef __cplusplus
extern "C" {
#endif

#define UVS_MAX_PORTS 18   /* NVLink 5 links of one B200 */
#define UVS_MAX_MEMBERS 8  /* physical devices behind one aggregation device */
#define UVS_MAX_PATHS 32
#define UVS_MAX_NODES 64

typedef enum uvs_topo_type { UVS_TOPO_FULLMESH = 0, UVS_TOPO_CLOS_PLANES = 1 } uvs_topo_type_t;
typedef enum uvs_tp_type { UVS_RTP = 0, UVS_CTP = 1, UVS_UTP = 2 } uvs_tp_type_t;

typedef struct uvs_agg_dev {
  urma_eid_t agg_eid;
  char name[64];
  uint32_t member_num;
  urma_eid_t member_eids[UVS_MAX_MEMBERS];
  char member_names[UVS_MAX_MEMBERS][64];
} uvs_agg_dev_t;

typedef struct uvs_topo_node {
  uint32_t type;        /* uvs_topo_type_t */
  uint32_t super_node_id;
  uint32_t node_id;
  uint32_t is_current;  /* this process runs on the node */
  uint32_t port_num;
  /* FULLMESH: bit r of links[p] = port p is wired to node r. CLOS_PLANES: port p belongs to plane p (all nodes). */
  uint64_t links[UVS_MAX_PORTS];
  urma_eid_t primary_eid;
  urma_eid_t port_eids[UVS_MAX_PORTS];
} uvs_topo_node_t;

typedef struct uvs_path {
  uint32_t src_node, dst_node;
  uint32_t src_port, dst_port;
  urma_eid_t src_eid, dst_eid;
} uvs_path_t;

typedef struct uvs_path_set {
  uint32_t topo_type;
  uint32_t path_count;
  uvs_path_t paths[UVS_MAX_PATHS];
} uvs_path_set_t;

/* aggregation devices */
URMA_EXPORT int uvs_create_agg_dev(const urma_eid_t* agg_eid, const char* dev_name, const char* const* member_names,
                                   uint32_t member_num);
URMA_EXPORT int uvs_delete_agg_dev(const urma_eid_t* agg_eid);
URMA_EXPORT int uvs_get_agg_dev(const char* dev_name, uvs_agg_dev_t* out);
URMA_EXPORT int uvs_get_device_name_by_eid(const urma_eid_t* eid, char* buf, size_t len);

/* topology */
URMA_EXPORT int uvs_set_topo_info(const uvs_topo_node_t* nodes, uint32_t node_num);
URMA_EXPORT int uvs_get_topo_info(uvs_topo_node_t* nodes, uint32_t max_nodes, uint32_t* node_num);
/* builds the topology of this host from the URMA device list: every `cudaN` device is a node of an NVSwitch Clos with
 * UVS_MAX_PORTS planes, every `shmN` device a node of a full mesh. Returns the number of nodes. */
URMA_EXPORT int uvs_discover_local_topology(void);

/* primary-entity table: which main EID owns a (port / virtual) EID */
URMA_EXPORT int uvs_insert_main_ue_eid(const urma_eid_t* eid, const urma_eid_t* main_ue_eid);
URMA_EXPORT int uvs_insert_main_ue_eid_batch(const urma_eid_t* main_ue_eid, const urma_eid_t* eids, uint32_t eid_num);
URMA_EXPORT int uvs_delete_main_ue_eid(const urma_eid_t* eid);
URMA_EXPORT int uvs_lookup_main_ue_eid(const urma_eid_t* eid, urma_eid_t* main_ue_eid);
URMA_EXPORT int uvs_flush_main_ue_eid(void);

/* every (source port, destination port) pair that connects the nodes owning the two EIDs (primary, port or main-UE
 * mapped EIDs are accepted). Returns 0 and fills `out`, or a negative errno value. */
URMA_EXPORT int uvs_get_path_set(const urma_eid_t* src_eid, const urma_eid_t* dst_eid, uvs_tp_type_t tp_type,
                                 uvs_path_set_t* out);

#ifdef __cplusplus
}
#endif
#endif
