"""Import alias: the reference's native module name (``import schemoe_custom_kernel``)."""
from planmoe_b200.custom import *  # noqa: F401,F403
from planmoe_b200.custom import (clear_ptr_lst, compress_operation, comm_operation,  # noqa: F401
                                 decompress_operation, init_nccl, get_nccl_unique_id,
                                 get_nccl_unique_id_size, invoke, inject_source, invoke_cpu_fp32,
                                 invoke_cpu_fp64, update_sdk_home)
