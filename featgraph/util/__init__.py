from featgraph_b200.util import util_convert_csr_to_dds, util_partition_adj_coo_2d  # noqa: F401
