#!/usr/bin/env bash
# Launch a training job on one node, one process per GPU (same environment surface as the reference's
# run_train.sh: NGPU, LOG_RANK, MODULE, CONFIG, COMM_MODE; extra arguments are passed through as config overrides).
#
#   NGPU=8 MODULE=llama3 CONFIG=llama3_8b ./run_train.sh --training.steps 100
#   COMM_MODE=fake_backend NGPU=64 ./run_train.sh          # config validation on one process, no collectives run
set -euo pipefail

NGPU=${NGPU:-8}
LOG_RANK=${LOG_RANK:-0}
MODULE=${MODULE:-llama3}
CONFIG=${CONFIG:-llama3_debugmodel}
COMM_MODE=${COMM_MODE:-}
TRAIN_FILE=${TRAIN_FILE:-torchtitan_b200.train}
MASTER_PORT=${MASTER_PORT:-29500}

export PYTORCH_ALLOC_CONF=${PYTORCH_ALLOC_CONF:-expandable_segments:True}
cd "$(dirname "$0")"

if [ -n "$COMM_MODE" ]; then
    # one process stands in for NGPU ranks: meshes, sharding plans and configs are built, no GPU communication runs
    echo "Running with comm.mode=${COMM_MODE} for a world of ${NGPU} ranks"
    NGPU="$NGPU" LOCAL_RANK=0 python -m "${TRAIN_FILE}" --module "${MODULE}" --config "${CONFIG}" \
        --comm.mode "${COMM_MODE}" --training.steps 1 "$@"
else
    python -m torch.distributed.run --nnodes=1 --nproc-per-node="${NGPU}" --master-addr 127.0.0.1 \
        --master-port "${MASTER_PORT}" --local-ranks-filter "${LOG_RANK}" --role rank --tee 3 \
        -m "${TRAIN_FILE}" --module "${MODULE}" --config "${CONFIG}" "$@"
fi
