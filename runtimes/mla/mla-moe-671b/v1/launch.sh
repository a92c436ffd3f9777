#!/bin/sh
# Launch the default profile of this recipe version (eight ranks, one per GPU) with the site file given as $1.
set -eu
here=$(cd "$(dirname "$0")/../../../.." && pwd)
cd "$here"
cmd=$(python -m rexl3_b200.recipes --root runtimes --family mla --model mla-moe-671b --version v1 --site "$1" | sed 's/^[^ ]* -m rexl3_b200.server//')
exec env NCCL_NVLS_ENABLE=0 python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29600 -m rexl3_b200.server $cmd
