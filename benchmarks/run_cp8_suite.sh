#!/usr/bin/env bash
# Full-box (8 GPU) measurement suite: correctness script, exchange micro-benchmark (with o_proj paths),
# decode-step benchmark at batch 8 / 32 (both arms, one-kernel path), MLA fp8 decode step (both arms), device timelines.  Usage: benchmarks/run_cp8_suite.sh OUTDIR [N]
set -u
cd "$(dirname "$0")/.."
OUT=${1:-results/cp8}
N=${2:-8}
mkdir -p "$OUT"
TR="python -m torch.distributed.run --nnodes=1 --nproc-per-node=$N --master-addr 127.0.0.1"
run() { local name=$1; shift; echo "== $name"; timeout 600 "$@" > "$OUT/$name.log" 2>&1; echo "   rc=$?"; grep '^{' "$OUT/$name.log" > "$OUT/$name.json" || true; }
run tests $TR --master-port 29701 tests/multi_gpu/run_exchange.py
grep -E "FAIL|ALL PASSED" "$OUT/tests.log" | tail -3
run exchange $TR --master-port 29702 benchmarks/exchange_bench.py --tokens 1,8,32,128,256,512 --mode graph --per-op
run exchange_oproj $TR --master-port 29703 benchmarks/exchange_bench.py --shapes gqa --tokens 1,8,32,64,256 --mode graph --with-oproj \
    --paths helix_fused,oproj:helix_one_kernel,oproj:helix_two_kernels,oproj:helix_exchange_auto_gemm,oproj:reference_linear,oproj:nccl_torch_linear
run decode_b8 $TR --master-port 29704 bench.py --gpus $N --steps 10 --warmup 3
run decode_b8_ref $TR --master-port 29707 bench.py --impl reference --gpus $N --steps 10 --warmup 3
run decode_b8_one_kernel $TR --master-port 29708 bench.py --gpus $N --steps 10 --warmup 3 --fuse-oproj auto
run decode_b32_l20 $TR --master-port 29705 bench.py --gpus $N --steps 10 --warmup 3 --batch-per-gpu 4 --layers 20
run decode_b32_l20_ref $TR --master-port 29709 bench.py --impl reference --gpus $N --steps 10 --warmup 3 --batch-per-gpu 4 --layers 20
run mla_b32_l8 $TR --master-port 29706 benchmarks/mla_decode_bench.py --ctx 1048576 --batch 32 --layers 8 --steps 5
run mla_b32_l8_ref $TR --master-port 29710 benchmarks/mla_decode_bench.py --ctx 1048576 --batch 32 --layers 8 --steps 5 --impl reference --ref-dtype fp8
HELIX_A2A_EXCHANGE_TRACE=1 run exchange_timeline $TR --master-port 29711 benchmarks/exchange_timeline.py --shape gqa --tokens 1,8,64,256
HELIX_A2A_EXCHANGE_TRACE=1 run one_kernel_timeline $TR --master-port 29712 benchmarks/fused_timeline.py --tokens 1,8,32,64 --hidden 8192
echo done
