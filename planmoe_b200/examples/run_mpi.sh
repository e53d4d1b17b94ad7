#!/bin/bash
# Two hosts x LOCAL_SIZE GPUs under OpenMPI; on one 8-GPU NVSwitch box LOCAL_SIZE=4 gives the two
# logical 4-GPU groups that the pipe / hetu / dd algorithms distinguish.
#   HOSTS=a,b LOCAL_SIZE=8 MASTER_ADDR=a ./run_mpi.sh --encode int8 --comm pipe
HOSTS=${HOSTS:-localhost}
LOCAL_SIZE=${LOCAL_SIZE:-8}
mpiexec -bind-to none -host ${HOSTS} -x LOCAL_SIZE=${LOCAL_SIZE} -x MASTER_ADDR=${MASTER_ADDR:-127.0.0.1} \
    -x NCCL_DEBUG=WARN python3 -m planmoe_b200.launcher.run -m planmoe_b200.examples.pre_test "$@"
