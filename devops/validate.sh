#!/usr/bin/env bash
# Tiered validation: tier 1 needs no GPU (build + CPU tests), tier 2 runs the GPU tests, tier 3 the
# multi-GPU tests and a short benchmark on all GPUs of the node.
set -euo pipefail
cd "$(dirname "$0")/.."
TIER="${1:-1}"
python devops/warm_kernels.py --check-env --compile
python -m pytest tests -x -q -m "not gpu"
if [[ "$TIER" -ge 2 ]]; then
  python -m pytest tests -x -q -m gpu
  python bench.py --steps 50 --warmup 3
fi
if [[ "$TIER" -ge 3 ]]; then
  N="$(python -c 'import torch; print(torch.cuda.device_count())')"
  NCCL_NVLS_ENABLE=0 python -m torch.distributed.run --nnodes=1 --nproc-per-node "$N" --master-addr 127.0.0.1 \
      bench.py --gpus "$N" --steps 100 --warmup 5
fi
