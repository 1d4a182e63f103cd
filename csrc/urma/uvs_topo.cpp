// In-process topology / aggregation-device registry. See uvs_topo.h.
#include "uvs_topo.h"

#include <errno.h>
#include <stdio.h>
#include <string.h>

#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "urma_api.h"

namespace {

struct EidKey {
  uint8_t raw[URMA_EID_SIZE];
  bool operator<(const EidKey& o) const { return memcmp(raw, o.raw, URMA_EID_SIZE) < 0; }
};
EidKey key_of(const urma_eid_t* e) {
  EidKey k;
  memcpy(k.raw, e->raw, URMA_EID_SIZE);
  return k;
}

struct Registry {
  std::mutex mu;
  std::map<EidKey, uvs_agg_dev_t> agg;           // by aggregation EID
  std::vector<uvs_topo_node_t> nodes;
  std::map<EidKey, EidKey> main_ue;              // eid -> main entity eid
};
Registry& reg() {
  static Registry* r = new Registry();
  return *r;
}

// node index that owns `eid` (primary or port EID), following the main-UE table once; -1 if unknown
int node_of(Registry& r, const urma_eid_t* eid) {
  EidKey k = key_of(eid);
  auto it = r.main_ue.find(k);
  if (it != r.main_ue.end()) k = it->second;
  for (size_t i = 0; i < r.nodes.size(); ++i) {
    const uvs_topo_node_t& n = r.nodes[i];
    if (memcmp(n.primary_eid.raw, k.raw, URMA_EID_SIZE) == 0) return (int)i;
    for (uint32_t p = 0; p < n.port_num && p < UVS_MAX_PORTS; ++p)
      if (memcmp(n.port_eids[p].raw, k.raw, URMA_EID_SIZE) == 0) return (int)i;
  }
  return -1;
}

}  // namespace

extern "C" {

int uvs_create_agg_dev(const urma_eid_t* agg_eid, const char* dev_name, const char* const* member_names,
                       uint32_t member_num) {
  if (!agg_eid || !dev_name || !member_names || member_num == 0 || member_num > UVS_MAX_MEMBERS) return -EINVAL;
  uvs_agg_dev_t d;
  memset(&d, 0, sizeof(d));
  d.agg_eid = *agg_eid;
  snprintf(d.name, sizeof(d.name), "%s", dev_name);
  d.member_num = member_num;
  for (uint32_t i = 0; i < member_num; ++i) {
    if (!member_names[i]) return -EINVAL;
    snprintf(d.member_names[i], sizeof(d.member_names[i]), "%s", member_names[i]);
    if (urma_device_t* dev = urma_get_device_by_name(member_names[i])) d.member_eids[i] = dev->eid;
  }
  Registry& r = reg();
  std::lock_guard<std::mutex> l(r.mu);
  for (auto& kv : r.agg)
    if (strcmp(kv.second.name, dev_name) == 0) return -EEXIST;
  if (!r.agg.emplace(key_of(agg_eid), d).second) return -EEXIST;
  return 0;
}

int uvs_delete_agg_dev(const urma_eid_t* agg_eid) {
  if (!agg_eid) return -EINVAL;
  Registry& r = reg();
  std::lock_guard<std::mutex> l(r.mu);
  return r.agg.erase(key_of(agg_eid)) ? 0 : -ENOENT;
}

int uvs_get_agg_dev(const char* dev_name, uvs_agg_dev_t* out) {
  if (!dev_name || !out) return -EINVAL;
  Registry& r = reg();
  std::lock_guard<std::mutex> l(r.mu);
  for (auto& kv : r.agg) {
    if (strcmp(kv.second.name, dev_name) == 0) {
      *out = kv.second;
      return 0;
    }
  }
  return -ENOENT;
}

int uvs_get_device_name_by_eid(const urma_eid_t* eid, char* buf, size_t len) {
  if (!eid || !buf || len == 0) return -EINVAL;
  {
    Registry& r = reg();
    std::lock_guard<std::mutex> l(r.mu);
    auto it = r.agg.find(key_of(eid));
    if (it != r.agg.end()) {
      snprintf(buf, len, "%s", it->second.name);
      return 0;
    }
  }
  if (urma_device_t* d = urma_get_device_by_eid(*eid)) {
    snprintf(buf, len, "%s", d->name);
    return 0;
  }
  return -ENOENT;
}

int uvs_set_topo_info(const uvs_topo_node_t* nodes, uint32_t node_num) {
  if ((!nodes && node_num) || node_num > UVS_MAX_NODES) return -EINVAL;
  uint32_t current = 0;
  for (uint32_t i = 0; i < node_num; ++i) {
    if (nodes[i].port_num > UVS_MAX_PORTS || nodes[i].type > UVS_TOPO_CLOS_PLANES) return -EINVAL;
    current += nodes[i].is_current ? 1 : 0;
  }
  if (node_num && current != 1) return -EINVAL;  // exactly one node is "here"
  Registry& r = reg();
  std::lock_guard<std::mutex> l(r.mu);
  r.nodes.assign(nodes, nodes + node_num);
  return 0;
}

int uvs_get_topo_info(uvs_topo_node_t* nodes, uint32_t max_nodes, uint32_t* node_num) {
  if (!node_num) return -EINVAL;
  Registry& r = reg();
  std::lock_guard<std::mutex> l(r.mu);
  *node_num = (uint32_t)r.nodes.size();
  if (!nodes) return 0;
  if (max_nodes < r.nodes.size()) return -ENOSPC;
  for (size_t i = 0; i < r.nodes.size(); ++i) nodes[i] = r.nodes[i];
  return 0;
}

int uvs_discover_local_topology(void) {
  int n = 0;
  urma_device_t** list = urma_get_device_list(&n);
  std::vector<uvs_topo_node_t> nodes;
  bool have_current = false;
  for (int i = 0; i < n && nodes.size() < UVS_MAX_NODES; ++i) {
    const urma_device_t* d = list[i];
    const bool gpu = strncmp(d->name, "cuda", 4) == 0;
    const bool shm = strncmp(d->name, "shm", 3) == 0;
    if (!gpu && !shm) continue;  // virtual devices (bond) are aggregation devices, not nodes
    uvs_topo_node_t t;
    memset(&t, 0, sizeof(t));
    t.type = gpu ? UVS_TOPO_CLOS_PLANES : UVS_TOPO_FULLMESH;
    t.node_id = (uint32_t)nodes.size();
    t.primary_eid = d->eid;
    t.port_num = gpu ? UVS_MAX_PORTS : 1;
    for (uint32_t p = 0; p < t.port_num; ++p) {
      t.port_eids[p] = d->eid;
      t.port_eids[p].raw[14] = (uint8_t)(p + 1);  // port EIDs differ from the primary in one byte
      t.links[p] = ~0ull;                         // every plane / the mesh reaches every node
    }
    if (!have_current) {
      t.is_current = 1;
      have_current = true;
    }
    nodes.push_back(t);
  }
  if (list) urma_free_device_list(list);
  if (nodes.empty()) return 0;
  const int rc = uvs_set_topo_info(nodes.data(), (uint32_t)nodes.size());
  return rc ? rc : (int)nodes.size();
}

int uvs_insert_main_ue_eid(const urma_eid_t* eid, const urma_eid_t* main_ue_eid) {
  if (!eid || !main_ue_eid) return -EINVAL;
  Registry& r = reg();
  std::lock_guard<std::mutex> l(r.mu);
  return r.main_ue.emplace(key_of(eid), key_of(main_ue_eid)).second ? 0 : -EEXIST;
}
int uvs_insert_main_ue_eid_batch(const urma_eid_t* main_ue_eid, const urma_eid_t* eids, uint32_t eid_num) {
  if (!main_ue_eid || (!eids && eid_num)) return -EINVAL;
  Registry& r = reg();
  std::lock_guard<std::mutex> l(r.mu);
  for (uint32_t i = 0; i < eid_num; ++i)
    if (r.main_ue.count(key_of(&eids[i]))) return -EEXIST;  // all or nothing
  for (uint32_t i = 0; i < eid_num; ++i) r.main_ue.emplace(key_of(&eids[i]), key_of(main_ue_eid));
  return 0;
}
int uvs_delete_main_ue_eid(const urma_eid_t* eid) {
  if (!eid) return -EINVAL;
  Registry& r = reg();
  std::lock_guard<std::mutex> l(r.mu);
  return r.main_ue.erase(key_of(eid)) ? 0 : -ENOENT;
}
int uvs_lookup_main_ue_eid(const urma_eid_t* eid, urma_eid_t* main_ue_eid) {
  if (!eid || !main_ue_eid) return -EINVAL;
  Registry& r = reg();
  std::lock_guard<std::mutex> l(r.mu);
  auto it = r.main_ue.find(key_of(eid));
  if (it == r.main_ue.end()) return -ENOENT;
  memcpy(main_ue_eid->raw, it->second.raw, URMA_EID_SIZE);
  return 0;
}
int uvs_flush_main_ue_eid(void) {
  Registry& r = reg();
  std::lock_guard<std::mutex> l(r.mu);
  r.main_ue.clear();
  return 0;
}

int uvs_get_path_set(const urma_eid_t* src_eid, const urma_eid_t* dst_eid, uvs_tp_type_t tp_type,
                     uvs_path_set_t* out) {
  if (!src_eid || !dst_eid || !out || tp_type > UVS_UTP) return -EINVAL;
  Registry& r = reg();
  std::lock_guard<std::mutex> l(r.mu);
  const int s = node_of(r, src_eid), d = node_of(r, dst_eid);
  if (s < 0 || d < 0) return -ENOENT;
  const uvs_topo_node_t& a = r.nodes[s];
  const uvs_topo_node_t& b = r.nodes[d];
  if (a.type != b.type) return -EHOSTUNREACH;
  memset(out, 0, sizeof(*out));
  out->topo_type = a.type;
  auto add = [&](uint32_t sp, uint32_t dp) {
    if (out->path_count >= UVS_MAX_PATHS) return;
    uvs_path_t& p = out->paths[out->path_count++];
    p.src_node = a.node_id;
    p.dst_node = b.node_id;
    p.src_port = sp;
    p.dst_port = dp;
    p.src_eid = a.port_eids[sp];
    p.dst_eid = b.port_eids[dp];
  };
  if (a.type == UVS_TOPO_CLOS_PLANES) {
    // plane p connects port p of every node that has it
    for (uint32_t p = 0; p < a.port_num && p < b.port_num; ++p)
      if ((a.links[p] >> (b.node_id & 63)) & 1 && (b.links[p] >> (a.node_id & 63)) & 1) add(p, p);
  } else {
    for (uint32_t sp = 0; sp < a.port_num; ++sp) {
      if (!((a.links[sp] >> (b.node_id & 63)) & 1)) continue;
      for (uint32_t dp = 0; dp < b.port_num; ++dp)
        if ((b.links[dp] >> (a.node_id & 63)) & 1) add(sp, dp);
    }
  }
  return out->path_count ? 0 : -EHOSTUNREACH;
}

}  // extern "C"
