"""Max-vertex-value on GPUs (device path of
alg/graph_alg/max_vertex_value/max_vertex_value.hpp:70-121 and of its Pregel form,
max_vertex_value_pregel.cpp:28-53).

``MvvGpu`` is the vertex program ``MaxValueVertices`` of ``paracel_b200.pregel_gpu``: the value
of vertex v is the scalar key ``<v>`` of a table sharded over the ranks' HBM with the
``max_updater`` handler.  A superstep pushes the value of every active local vertex to its
out-neighbours (``paracel_bupdate_multi`` = system-scope atomic max at the owner),
synchronises, reads the owned values back and keeps the vertices whose value changed active;
the run ends when no vertex changed anywhere."""
from __future__ import annotations

from ..pregel_gpu import MaxValueVertices


class MvvGpu(MaxValueVertices):
    def __init__(self, n_vertices: int, group=None, device=None, comm=None, hosts_dct_str=None,
                 output: str = "", names=None, update_func: str = "max_updater"):
        from ..ps.device_handlers import resolve_device_handler
        if resolve_device_handler(update_func).kind != "max":
            raise ValueError("max-vertex-value needs a max handler")
        super().__init__(n_vertices, group=group, device=device, comm=comm, hosts_dct_str=hosts_dct_str,
                         output=output, names=names)

    def solve(self, max_rounds: int = 1 << 20) -> int:
        return self.run_supersteps(max_rounds)
