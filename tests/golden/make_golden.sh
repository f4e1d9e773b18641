#!/bin/bash
# Usage: make_golden.sh PATH_TO_THE_REFERENCE_CHECKOUT
# Builds the reference's CPU sources (a read-only checkout) and runs ref_driver.c, ref_driver2.c and ref_sampler.c
# against them; writes logits.bin, logits2.bin, route.bin and samples.bin next to this script.  No network, no GPU.
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
gcc -O2 -std=c11 -I$R/include "$HERE/ref_driver2.c" "$W/libtq.a" -lm -lpthread -o "$W/ref_driver2"
gcc -O2 -std=c11 -I$R/include "$HERE/ref_sampler.c" "$W/libtq.a" -lm -lpthread -o "$W/ref_sampler"
(cd "$W" && ./ref_driver && ./ref_driver2 && ./ref_sampler)
for f in logits.bin logits2.bin route.bin samples.bin; do cp "$W/$f" "$HERE/$f"; done
rm -rf "$W"
echo "wrote logits.bin, logits2.bin, route.bin and samples.bin in $HERE"
