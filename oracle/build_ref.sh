#!/bin/bash
# Test infrastructure, not product code.
# Compiles the reference's own CPU implementation of the training step (its Neural_Network sources and the
# Common_Library helpers they need) from where they lie in the read-only reference checkout into
# oracle/_ref/libmyea_ref.so, together with oracle/ref_harness.cpp (a C-ABI driver) and oracle/ref_stubs.cpp.
# No reference source is copied into the repository: BOM-stripped copies live only in oracle/_ref/build.
#   usage: oracle/build_ref.sh [reference checkout]     (without the argument: the checkout the container mounts)
#          SCALAR=double oracle/build_ref.sh ...        the same sources with the reference's COMPILE_DOUBLE switch
#                                                       (its scalar type becomes double) -> oracle/_ref/libmyea_ref_f64.so,
#                                                       the tie-breaker where the fp32 reference and the GPU differ
# Nothing is built (exit 0) when the checkout is absent; a prebuilt oracle/_ref/libmyea_ref*.so is used as is.
set -e
HERE=$(cd "$(dirname "$0")" && pwd)
REF=${1:-/root/reference}
OUT=$HERE/_ref
if [ ! -d "$REF/Neural_Network_Library_Windows" ]; then echo "build_ref: no reference checkout at $REF, nothing built"; exit 0; fi
NN=$REF/Neural_Network_Library_Windows
SCALAR=${SCALAR:-float}
if [ "$SCALAR" = double ]; then W=$OUT/build_f64; LIB=libmyea_ref_f64.so; TYPE=-DCOMPILE_DOUBLE; else W=$OUT/build; LIB=libmyea_ref.so; TYPE=-DCOMPILE_FLOAT; fi
mkdir -p $W/src $W/obj $W/cobj $W/csrc
FLAGS="-std=c++17 -fopenmp -O3 -march=x86-64-v3 -w -fPIC -fpermissive -include cfloat -DCOMPILE_x64 $TYPE -DCOMPILE_LINUX -DCOMPILE_COUT -I $HERE/shim -I $REF/Common_Library/include -I $NN/Header_Files -I $HERE/../include ${EXTRA_FLAGS}"
# stale or un-buildable translation units (no matching declarations, or Eigen)
SKIP="Randomize|Xavier|Neural_Network__Orthogonal|Tied_Parameter|Tied_Weight|Initialization__Orthogonal"
for f in $NN/Source_Files/Neural_Network/*.cpp; do
  b=$(basename $f .cpp); echo $b | grep -Eq "$SKIP" && continue
  [ $W/obj/$b.o -nt $f ] && continue
  sed 's/\xEF\xBB\xBF//g' "$f" > $W/src/$b.cpp; echo $b
done > $W/todo.txt
cat $W/todo.txt | xargs -r -P $(nproc) -I{} g++ $FLAGS -c $W/src/{}.cpp -o $W/obj/{}.o
for f in $(cd $REF/Common_Library/src && find . -name '*.cpp' | grep -Ev "Windows|Strings/String.cpp|Shutdown|Reallocate"); do
  o=$(echo $f | tr '/' '_' | sed 's/^\._//;s/\.cpp$//')
  [ $W/cobj/$o.o -nt $REF/Common_Library/src/$f ] && continue
  sed 's/\xEF\xBB\xBF//g' $REF/Common_Library/src/$f > $W/csrc/$o.cpp; echo $o
done > $W/ctodo.txt
cat $W/ctodo.txt | xargs -r -P $(nproc) -I{} g++ $FLAGS -c $W/csrc/{}.cpp -o $W/cobj/{}.o
g++ $FLAGS -shared $HERE/ref_harness.cpp $HERE/ref_stubs.cpp $W/obj/*.o $W/cobj/*.o -o $OUT/$LIB
echo "build_ref: built $OUT/$LIB"
