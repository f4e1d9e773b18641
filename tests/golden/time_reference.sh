#!/bin/bash
# Usage: time_reference.sh PATH_TO_THE_REFERENCE_CHECKOUT [THREADS]
# Builds the reference's CPU sources and times its own forward (ref_timing.c) on models of 1 and 2 layers with the
# layer sizes of Qwen1.5-MoE-A2.7B; writes reference_cpu_timing.txt next to this script.  No network, no GPU.
set -e
R=${1:?path of the reference checkout}
T=${2:-$(nproc)}
HERE=$(cd "$(dirname "$0")" && pwd)
W=$(mktemp -d)
for f in $R/src/core/*.c $R/src/cache/*.c $R/src/backend/cpu/*.c $R/src/engine/*.c; do
  gcc -O2 -std=c11 -D_GNU_SOURCE -D__fp16=_Float16 -I$R/include -c "$f" -o "$W/$(basename "$f" .c).o"
done
ar rcs "$W/libtq.a" "$W"/*.o
gcc -O2 -std=c11 -D_GNU_SOURCE -I$R/include "$HERE/ref_timing.c" "$W/libtq.a" -lm -lpthread -o "$W/ref_timing"
{
  echo "# reference tq_forward on the CPU of this machine ($(nproc) cores: $(grep -m1 'model name' /proc/cpuinfo | cut -d: -f2 | xargs)), float32, one token at a time"
  "$W/ref_timing" 1 "$T"
  "$W/ref_timing" 2 "$T"
} | tee "$HERE/reference_cpu_timing.txt"
rm -rf "$W"
