"""umdk_b200: a Blackwell-native (sm_100a, NVLink 5 / NVSwitch) memory-semantic communication and serving
acceleration framework with the capabilities of UMDK: URMA-style remote memory API, expert-parallel MoE
dispatch / combine / fused MoE kernels, tensor-parallel fused GEMM+collective kernels, sparse MLA decode attention
and KV-cache offload, plus UMQ / URPC / DLock / socket-shim services on the host side."""
from .buffer import Buffer, Config, EventOverlap  # noqa: F401

__version__ = "0.1.0"


def load_torch_ops():
    """Registers `torch.ops.umdk_cam_op_lib.*` (idempotent)."""
    from .ops import cam_ops  # noqa: F401
    return cam_ops
