#!/usr/bin/env bash
# CPU-only continuous-integration job: build the native library and run the CPU test suite once per assertion mode,
# then the host runtime's self-test under AddressSanitizer+UBSan and under ThreadSanitizer.
#
# The reference runs its whole suite twice, with assertions compiled out and in
# (.github/workflows/standard_library_tests_and_examples.yml:24-31, stdlib/test/lit.cfg.py:70-75); here the switch is
# the -DB2_ASSERT_MODE value the kernels and the runtime are compiled with: 0 none, 2 safe (the default), 3 all.
# GPU tests (`-m gpu`) need a B200 and are not part of this job.
#
#   ./ci.sh            all modes
#   ./ci.sh 2          one mode
set -euo pipefail
cd "$(dirname "$0")"
modes=("$@")
if [ ${#modes[@]} -eq 0 ]; then modes=(0 3 2); fi   # the default mode last, so the tree is left built with it
for mode in "${modes[@]}"; do
  echo "== B2_ASSERT_MODE=${mode}: build"
  python -m mojo_b200.build --clean --assert-mode "${mode}"
  echo "== B2_ASSERT_MODE=${mode}: pytest -m 'not gpu'"
  B2_ASSERT_MODE="${mode}" python -m pytest tests/ -x -q -m "not gpu"
done
echo "== host runtime self-test under sanitizers"
python -m mojo_b200.build --selftest address
python -m mojo_b200.build --selftest thread
echo "ci: ok"
