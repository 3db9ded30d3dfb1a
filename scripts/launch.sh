#!/usr/bin/env bash
# Elastic launcher: torchrun with restarts; the rendezvous backend and endpoint come from the YAML config
# (elastic.rdzv_backend / elastic.rdzv_endpoint) unless RDZV_BACKEND / RDZV_ENDPOINT are set.
#   scripts/launch.sh configs/olmoe_1b7b.yaml [nproc_per_node] [nnodes] [extra train.py flags...]
set -euo pipefail
CONFIG="${1:?usage: launch.sh <config.yaml> [nproc_per_node] [nnodes] [train.py flags]}"
NPROC="${2:-$(python -c 'import torch; print(max(torch.cuda.device_count(), 1))')}"
NNODES="${3:-1}"
shift $(( $# < 3 ? $# : 3 ))
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")/.." && pwd)"
read_yaml() { python - "$CONFIG" "$1" "$2" <<'PY'
import sys, yaml
cfg = yaml.safe_load(open(sys.argv[1])) or {}
print((cfg.get("elastic") or {}).get(sys.argv[2], sys.argv[3]))
PY
}
RDZV_BACKEND="${RDZV_BACKEND:-$(read_yaml rdzv_backend c10d)}"
RDZV_ENDPOINT="${RDZV_ENDPOINT:-$(read_yaml rdzv_endpoint 127.0.0.1:29400)}"
RDZV_ID="${RDZV_ID:-cmoe-$(date +%s)}"
MAX_RESTARTS="${MAX_RESTARTS:-3}"
export RDZV_BACKEND RDZV_ENDPOINT RDZV_ID
export TORCH_NCCL_ASYNC_ERROR_HANDLING=1
if [ "$NNODES" = "1" ]; then
  exec python -m torch.distributed.run --standalone --local-addr 127.0.0.1 --nproc-per-node "$NPROC" \
       --max-restarts "$MAX_RESTARTS" "$HERE/train.py" --config "$CONFIG" "$@"
fi
exec python -m torch.distributed.run --nnodes "$NNODES" --nproc-per-node "$NPROC" --max-restarts "$MAX_RESTARTS" \
     --rdzv-backend "$RDZV_BACKEND" --rdzv-endpoint "$RDZV_ENDPOINT" --rdzv-id "$RDZV_ID" \
     "$HERE/train.py" --config "$CONFIG" "$@"
