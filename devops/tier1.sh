#!/usr/bin/env bash
# Image check on a build host without GPUs: build the image (which cross-compiles every sm_100a kernel), then run
# inside it the environment check, the CPU test suite, an import smoke, the entrypoint's dry run and a start-up
# without GPUs, which has to end with an application error (exit 1), not a hang, a crash of the container runtime
# or a success.  Every step's output and exit code is kept under $NAIVERT_VALIDATION_DIR.
set -euo pipefail
cd "$(dirname "$0")/.."
TAG="${1:-naivert-b200:tier1}"
OUT="${NAIVERT_VALIDATION_DIR:-$(pwd)/tests/results/tier1}"
DOCKER="${NAIVERT_DOCKER:-docker}"
mkdir -p "$OUT"
FAILED=0
run_step() {            # run_step NAME EXPECTED_EXIT CMD...
  local name="$1" want="$2" got=0
  shift 2
  echo "== $name"
  "$@" > "$OUT/$name.log" 2>&1 || got=$?
  echo "$got" > "$OUT/$name.exit"
  if [[ "$got" -ne "$want" ]]; then
    echo "FAILED: $name exited $got, expected $want (log: $OUT/$name.log)" >&2
    FAILED=1
    return 1
  fi
}
date -u +%FT%TZ > "$OUT/started"
run_step build 0 "$DOCKER" build -f devops/Dockerfile -t "$TAG" . || exit 1
in_image() { "$DOCKER" run --rm --entrypoint python "$TAG" "$@"; }
run_step checkenv 0 in_image devops/warm_kernels.py --check-env || true
run_step cputests 0 in_image -m pytest tests -x -q -m "not gpu" -p no:cacheprovider || true
run_step imports 0 in_image -c "import naivert_b200.runtime.session_engine, naivert_b200.serve.http, naivert_b200.prefill.native, naivert_b200.models.registry as r; print('imports ok', sorted(r.MODELS))" || true
run_step dryrun 0 "$DOCKER" run --rm -e NAIVERT_DRY_RUN=1 -e NAIVERT_MODEL=naive-n0.5 -e NAIVERT_MAX_DECODE_TOKENS=4096 "$TAG" || true
NAME="naivert-b200-tier1-$$"
trap '"$DOCKER" rm -f "$NAME" >/dev/null 2>&1 || true' EXIT
run_step nogpu 1 timeout 300 "$DOCKER" run --rm --name "$NAME" -e NAIVERT_GPUS=1 -e NAIVERT_RANDOM_INIT=1 "$TAG" || true
run_step compose 0 "$DOCKER" compose -f devops/docker-compose.yml config -q || true
run_step kernels 0 "$DOCKER" run --rm --entrypoint sh "$TAG" -c "ls -l naivert_b200/_lib" || true
"$DOCKER" image inspect "$TAG" --format '{{.Size}}' > "$OUT/size_bytes" 2>/dev/null || true
date -u +%FT%TZ > "$OUT/finished"
if [[ "$FAILED" -ne 0 ]]; then
  echo "TIER1_FAILED: logs in $OUT" >&2
  exit 1
fi
echo "TIER1_OK: logs in $OUT"
