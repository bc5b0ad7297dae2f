#!/usr/bin/env bash
# build_ref.sh -- TEST INFRASTRUCTURE ONLY.
#
# Compiles the reference's own HotSketch (tricks/sketch.cpp, read in place from the reference
# checkout, never copied into this repository) into oracle/_ref/libsketch_ref.so.  The source text is
# streamed through sed into the compiler with four mechanical fixes, each needed to make the
# reference usable as an oracle at all:
#   P1  drop the constructor's early return on an uninitialised member (sketch.cpp:50), which
#       otherwise leaves the tables unallocated;
#   P2  enlarge the static result arrays (sketch.cpp:10) from 16384 to 4 Mi entries so that a
#       65536-id call does not overflow them;
#   P3  allocate the main and LRU tables in one zeroed block, main table first (sketch.cpp:53-54),
#       so that reset()'s address tie-break (sketch.cpp:79-96) is the canonical order
#       main-before-LRU, bucket, slot instead of depending on the heap layout;
#   P4  make the class members visible to the state-dump shim (ref_shim.inc) appended below.
# Usage: build_ref.sh [reference_root]   (default: $CAFE_REFERENCE_ROOT, else the directory `reference`
# beside this repository; exits 0 and builds nothing when the reference checkout is absent, e.g. on a
# machine that only runs the prebuilt library).
set -euo pipefail
here="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
ref_root="${1:-${CAFE_REFERENCE_ROOT:-$here/../../reference}}"
src="$ref_root/tricks/sketch.cpp"
out_dir="$here/_ref"
if [ ! -f "$src" ]; then
    echo "build_ref.sh: $src not found; keeping any prebuilt $out_dir/libsketch_ref.so"
    exit 0
fi
mkdir -p "$out_dir"
# -march flags of the reference's own command (dlrm_s_pytorch.py:1402) are left out on purpose:
# the library must also run on the GPU box's host CPU, whose ISA is not known here.
{
    sed -e '/if (addr == NULL) return;/d' \
        -e 's/int ins\[16384\], que\[16384\];/int ins[1 << 22], que[1 << 22];/' \
        -e 's/^\( *\)b = new Bucket\[n1\];/\1{ char* blk = (char*)calloc(1, sizeof(Bucket) * (size_t)n1 + sizeof(Bucket2) * (size_t)n2 + 64); b = (Bucket*)blk; b2 = (Bucket2*)(blk + sizeof(Bucket) * (size_t)n1); }/' \
        -e '/b2 = new Bucket2\[n2\];/d' \
        -e 's/private:/public:/' \
        "$src"
    cat "$here/ref_shim.inc"
} | g++ -x c++ - -fPIC -shared --std=c++17 -O3 -o "$out_dir/libsketch_ref.so"
echo "built $out_dir/libsketch_ref.so"

# The one-stage sketch of the artifact tree (ArtifactEvaluation/embeddings/sketch.cpp), the same way: its static
# result arrays enlarged (:7), members made visible to the state-dump shim (ref_shim_sigmod.inc), nothing else.
src2="$ref_root/ArtifactEvaluation/embeddings/sketch.cpp"
if [ -f "$src2" ]; then
    {
        sed -e 's/int ins\[16384\], que\[16384\];/int ins[1 << 22], que[1 << 22];/' \
            -e 's/private:/public:/' \
            "$src2"
        cat "$here/ref_shim_sigmod.inc"
    } | g++ -x c++ - -fPIC -shared --std=c++17 -O3 -fopenmp -o "$out_dir/libsketch_sigmod_ref.so"
    echo "built $out_dir/libsketch_sigmod_ref.so"
fi
