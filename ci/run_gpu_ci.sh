#!/usr/bin/env bash
# GPU continuous-integration entry point for a machine with B200 GPUs.
#   1. build the sm_100a extension in-tree        2. one tiny forward+backward (smoke)
#   3. the GPU test-suite (multi-rank checks run when >= 2 GPUs are visible)
#   4. a short end-to-end benchmark step on a reduced model, to catch performance cliffs
# It never changes clocks, power limits or any other persistent GPU setting.
set -euo pipefail

ROOT="$(cd "$(dirname "${BASH_SOURCE[0]}")/.." && pwd)"
OUT="${CI_OUT:-$ROOT/ci_out}"
mkdir -p "$OUT"
cd "$ROOT"

echo "[ci] GPUs:"; nvidia-smi --query-gpu=index,name,memory.total --format=csv,noheader | tee "$OUT/gpus.txt"
NGPU=$(nvidia-smi --query-gpu=index --format=csv,noheader | wc -l)

echo "[ci] build"
python -c "import __graft_entry__ as g; g.build()" 2>&1 | tee "$OUT/build.log"

echo "[ci] smoke"
python -c "import __graft_entry__ as g; g.smoke()" 2>&1 | tee "$OUT/smoke.log"

echo "[ci] CPU suite"
python -m pytest tests -q -m "not gpu" 2>&1 | tee "$OUT/pytest_cpu.log"

echo "[ci] GPU suite on $NGPU GPU(s)"
NCCL_NVLS_ENABLE=0 python -m pytest tests -q -m gpu 2>&1 | tee "$OUT/pytest_gpu.log"

echo "[ci] short benchmark (4 layers, 64 completions)"
python bench.py --steps 2 --warmup 3 --dev-layers 4 --dev-group 64 2>&1 | tee "$OUT/bench_dev.log"
if [ "$NGPU" -ge 2 ]; then
  python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29561 \
    bench.py --gpus 2 --steps 2 --warmup 3 --dev-layers 4 --dev-group 64 2>&1 | tee "$OUT/bench_dev_2gpu.log"
fi
echo "[ci] done"
