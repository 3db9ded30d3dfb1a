#!/usr/bin/env bash
# Chaos helper: take one training worker down from the HOST (never by faulting a GPU).
#   scripts/simulate_node_failure.sh pod <pod-name> [namespace]     kubectl delete pod (k8s deployments)
#   scripts/simulate_node_failure.sh pid <pid>                      SIGKILL one local worker process
# TorchElastic (scripts/launch.sh, --max-restarts) relaunches the group; workers resume from the latest checkpoint.
set -euo pipefail
MODE="${1:?usage: simulate_node_failure.sh pod <name> [ns] | pid <pid>}"
case "$MODE" in
  pod)
    POD="${2:?pod name}"; NS="${3:-moe-engine}"
    echo "deleting pod $POD in namespace $NS (grace period 0)"
    kubectl delete pod "$POD" -n "$NS" --grace-period=0 --force
    ;;
  pid)
    PID="${2:?pid}"
    echo "sending SIGKILL to worker $PID"
    kill -9 "$PID"
    ;;
  *) echo "unknown mode $MODE" >&2; exit 2 ;;
esac
