#!/usr/bin/env bash
# Single-box launcher: one process per GPU over torch.distributed.run (NCCL is used for the bootstrap only).
#
#   bash launch.sh bench  N [extra bench.py flags]        headline benchmark on N GPUs (N = 1, 2, 4, 8)
#   bash launch.sh ref    N [extra flags]                 the same benchmark on the reference library (baseline/_ref)
#   bash launch.sh moe    N [extra bench_moe.py flags]    fused MoE forward / decode step / training step
#   bash launch.sh gemm   [extra bench_gemm.py flags]     grouped GEMM alone (one GPU)
#   bash launch.sh sweep  N                               normal-mode SM sweep that fills the per-rank-count config table
#   bash launch.sh test   [pytest args]                   GPU test suite (spawns its own ranks for the multi-GPU tests)
#
# The reference ships one sbatch file per experiment (deepep-efa-intranode.sbatch, deepep-efa-lowlatency*.sbatch); on a
# single box a plain launcher covers them.
set -euo pipefail
cd "$(dirname "${BASH_SOURCE[0]}")"
what=${1:-bench}
shift || true
port=${MASTER_PORT:-29533}

run_ranks() {  # run_ranks N script args...
    local n=$1
    shift
    if [ "$n" -eq 1 ]; then
        python "$@"
    else
        python -m torch.distributed.run --nnodes=1 --nproc-per-node "$n" --master-addr 127.0.0.1 --master-port "$port" "$@"
    fi
}

case "$what" in
    bench) n=${1:-1}; shift || true; run_ranks "$n" bench.py --gpus "$n" "$@" ;;
    ref) n=${1:-1}; shift || true; run_ranks "$n" bench.py --gpus "$n" --impl reference "$@" ;;
    moe) n=${1:-1}; shift || true; run_ranks "$n" bench_moe.py --gpus "$n" "$@" ;;
    gemm) python bench_gemm.py "$@" ;;
    sweep) n=${1:-8}; shift || true; run_ranks "$n" bench_normal_sweep.py --gpus "$n" "$@" ;;
    test) python -m pytest tests -m gpu -q "$@" ;;
    *) echo "usage: bash launch.sh bench|ref|moe|gemm|sweep|test ..." >&2; exit 2 ;;
esac
