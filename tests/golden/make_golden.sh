#!/bin/bash
# Usage: make_golden.sh PATH_TO_THE_REFERENCE_CHECKOUT
# Builds the reference's CPU sources (a read-only checkout) and runs ref_driver.c and ref_sampler.c against
# them; writes logits.bin and samples.bin next to this script.  No network, no GPU.
# The one flag the reference needs on x86-64 gcc is -D__fp16=_Float16 (src/engine/tq_transformer.c:3456).
set -e
R=${1:?path of the reference checkout}
HERE=$(cd "$(dirname "$0")" && pwd)
W=$(mktemp -d)
for f in $R/src/core/*.c $R/src/cache/*.c $R/src/backend/cpu/*.c $R/src/engine/*.c; do
  gcc -O2 -std=c11 -D_GNU_SOURCE -D__fp16=_Float16 -I$R/include -c "$f" -o "$W/$(basename "$f" .c).o"
done
ar rcs "$W/libtq.a" "$W"/*.o
gcc -O2 -std=c11 -I$R/include "$HERE/ref_driver.c" "$W/libtq.a" -lm -lpthread -o "$W/ref_driver"
gcc -O2 -std=c11 -I$R/include "$HERE/ref_sampler.c" "$W/libtq.a" -lm -lpthread -o "$W/ref_sampler"
(cd "$W" && ./ref_driver && ./ref_sampler)
cp "$W/logits.bin" "$HERE/logits.bin"
cp "$W/samples.bin" "$HERE/samples.bin"
rm -rf "$W"
echo "wrote $HERE/logits.bin and $HERE/samples.bin"
