#!/usr/bin/env bash
# Single-box sweep driver: exchange micro-benchmark, kernel benchmark and the decode-step benchmark
# for a list of CP degrees.  One JSON per point under $OUT; finished points are skipped unless
# FORCE=true (the reference's SLURM drivers resume the same way,
# benchmark/sbatch/run_gb200_aiperf_v3.sbatch:307-311).  DRY_RUN=true only prints the plan.
#
#   CP_DEGREES="2 4 8" TOKENS="1,8,32,128,256" MODE=graph OUT=results/sweep benchmarks/run_sweep.sh
set -u
cd "$(dirname "$0")/.."
CP_DEGREES=${CP_DEGREES:-"2 4 8"}
TOKENS=${TOKENS:-"1,8,32,128,256"}
MODE=${MODE:-graph}
OUT=${OUT:-results/sweep}
FORCE=${FORCE:-false}
DRY_RUN=${DRY_RUN:-false}
STEPS=${STEPS:-5}
PORT=${PORT:-29600}
export NCCL_NVLS_ENABLE=${NCCL_NVLS_ENABLE:-1}
mkdir -p "$OUT"

run_point() {   # name, command...
  local name=$1; shift
  local out="$OUT/$name.json"
  if [ -s "$out" ] && [ "$FORCE" != "true" ]; then echo "[skip] $name (exists)"; return 0; fi
  echo "[run ] $name: $*"
  [ "$DRY_RUN" = "true" ] && return 0
  if ! "$@" > "$OUT/$name.log" 2>&1; then echo "[fail] $name (see $OUT/$name.log)"; return 0; fi   # keep going
  grep '^{' "$OUT/$name.log" > "$out" || true
}

NGPU=$(nvidia-smi -L 2>/dev/null | wc -l)
run_point kernels python benchmarks/kernel_bench.py
for cp in $CP_DEGREES; do
  if [ "$DRY_RUN" != "true" ] && [ "$NGPU" -lt "$cp" ]; then echo "[skip] cp=$cp needs $cp GPUs"; continue; fi
  PORT=$((PORT + 1))
  run_point "exchange_cp${cp}" python -m torch.distributed.run --nnodes=1 --nproc-per-node "$cp" \
    --master-addr 127.0.0.1 --master-port "$PORT" benchmarks/exchange_bench.py --tokens "$TOKENS" --mode "$MODE"
  PORT=$((PORT + 1))
  run_point "decode_cp${cp}" python -m torch.distributed.run --nnodes=1 --nproc-per-node "$cp" \
    --master-addr 127.0.0.1 --master-port "$PORT" bench.py --gpus "$cp" --steps "$STEPS" --warmup 3
  PORT=$((PORT + 1))
  run_point "decode_ref_cp${cp}" python -m torch.distributed.run --nnodes=1 --nproc-per-node "$cp" \
    --master-addr 127.0.0.1 --master-port "$PORT" bench.py --impl reference --gpus "$cp" --steps "$STEPS" --warmup 3
done
echo "results in $OUT"
