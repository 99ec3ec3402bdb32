#!/bin/sh
# Compile the reference's own sm_100a modules (GPU parity oracle "O-so") from the
# sources where they lie in the read-only reference checkout.  Outputs go ONLY to
# oracle/_ref/ (git-ignored).  Nothing is copied from the reference: nvcc reads its
# two binding translation units in place.  Header-only third-party trees
# (tvm_ffi, the CUTLASS/CuTe + CCCL copies that ship inside the flashinfer wheel)
# come from the Python environment, exactly as the reference's build notes ask.
#
# This is test infrastructure: only tests/ and bench.py's reference comparison
# load what it produces.
set -eu
HERE=$(CDPATH= cd -- "$(dirname -- "$0")" && pwd)
REF=${LITEDSA_REFERENCE_DIR:-/root/reference}/kernels/b200/dsa
OUT=$HERE/_ref
PY=${PYTHON_BIN:-python3}
NVCC=${CUDA_HOME:-/usr/local/cuda}/bin/nvcc
[ -d "$REF" ] || { echo "reference checkout not present: $REF" >&2; exit 3; }
mkdir -p "$OUT"
TVM_INC=$($PY -c 'from pathlib import Path; import tvm_ffi; print(Path(tvm_ffi.__file__).parent / "include")')
FI=$($PY -c 'from pathlib import Path; import flashinfer; print(Path(flashinfer.__file__).parent / "data")')
PYINC=$($PY -c 'import sysconfig; print(sysconfig.get_path("include"))')
build_one() {  # $1 = binding .cu, $2 = output name
  "$NVCC" -shared --compiler-options=-fPIC --expt-relaxed-constexpr --expt-extended-lambda \
    -static-global-template-stub=false -std=c++17 -use_fast_math -O3 \
    -gencode=arch=compute_100a,code=sm_100a \
    -DPy_LIMITED_API=0x03090000 -D_GLIBCXX_USE_CXX11_ABI=1 \
    -DFLASHINFER_ENABLE_F16 -DFLASHINFER_ENABLE_BF16 -DFLASHINFER_ENABLE_FP8_E4M3 \
    -DFLASHINFER_ENABLE_FP8_E5M2 -DFLASHINFER_ENABLE_FP8_E8M0 -DFLASHINFER_ENABLE_FP4_E2M1 \
    -I"$REF" -I"$FI/cccl/cub" -I"$FI/cccl/libcudacxx/include" -I"$FI/cccl/thrust" \
    -I"$PYINC" -I"$TVM_INC" -I"$FI/cutlass/include" -I"$FI/cutlass/tools/util/include" \
    -I"$FI/include" -I"$FI/csrc" -I"$FI/spdlog/include" \
    "$REF/$1" -o "$OUT/$2.tmp" -L"${CUDA_HOME:-/usr/local/cuda}/lib64/stubs" -lcuda
  mv "$OUT/$2.tmp" "$OUT/$2"
  echo "built $OUT/$2"
}
build_one litedsa_jit_binding.cu litedsa_ref.so
build_one litedsa_dsv4_binding.cu litedsa_dsv4_ref.so
