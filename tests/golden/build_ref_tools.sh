#!/bin/sh
# Builds the reference's own compiler and probe tools straight from its source
# files with g++ (no build system), into a scratch directory outside both
# trees.  They are used ONLY to generate the golden fixtures committed beside
# this script (make_golden.py); nothing at test or run time needs them.
#
#   sh tests/golden/build_ref_tools.sh [REFERENCE_ROOT] [OUT_DIR]
#
# Produces OUT_DIR/seeml-update-compile, OUT_DIR/seeml-plan-probe and
# OUT_DIR/seeml-seeu-dump.  Flags are the ones the reference ships its runtime
# package with (-std=c++23 -O2, no -march=native), so no FMA contraction
# appears in any result.
set -eu
REF=${1:-/root/reference}
OUT=${2:-/tmp/see_ref_tools}
mkdir -p "$OUT/obj"
CXX=${CXX:-g++}
CXXFLAGS="-std=c++23 -O2 -pthread -I$REF -w"

PAR="source/parallel/parallel_for.cc"
SIR="compiler/frontend/representation/type.cc compiler/frontend/representation/value.cc
compiler/frontend/representation/operation.cc compiler/frontend/representation/block.cc
compiler/frontend/operator/convolution.cc compiler/frontend/operator/linear.cc
compiler/frontend/operator/normalization.cc compiler/frontend/operator/activation.cc
compiler/diagnostics/logger.cc"
TOK="source/tokenizer/byte_level_bpe.cc source/tokenizer/text_ingest.cc"
UPD="source/language/model_format.cc compiler/frontend/ingressor/model_reader.cc
compiler/frontend/ingressor/export_report.cc compiler/frontend/egressor/model_writer.cc
compiler/frontend/accountant/resource_analyzer.cc compiler/frontend/tokenization/corpus_ingress.cc
compiler/frontend/computation/value_resolver.cc compiler/frontend/topology/sema.cc
compiler/frontend/computation/parser.cc compiler/analysis/pass_manager.cc
compiler/analysis/topology/dce.cc compiler/analysis/algebra/epilogue_fuser.cc
compiler/analysis/algebra/rope_table.cc compiler/analysis/algebra/segment_mask.cc
compiler/analysis/algebra/chain_fuser.cc compiler/analysis/algebra/addend_fuser.cc
compiler/analysis/calculus/rematerializer.cc compiler/analysis/statistics/precision.cc
compiler/analysis/optimization/schedule.cc compiler/analysis/statistics/attention_tiling.cc
compiler/analysis/algebra/lora_grafter.cc compiler/analysis/algebra/merge_builder.cc
compiler/analysis/calculus/autodiff.cc compiler/analysis/optimization/optimizer.cc
compiler/analysis/statistics/quantization.cc compiler/backend/architecture/host_arch.cc
compiler/backend/architecture/kernel_policy_table.cc compiler/backend/allocation/arena_binder.cc
compiler/backend/assembly/plan_assembly.cc compiler/backend/selection/instruction_lowering.cc
compiler/driver/contract.cc compiler/driver/update_compiler.cc compiler/driver/statistics.cc
compiler/backend/packaging/native_emitter.cc"
RT="runtime/executor/gemm.cc runtime/executor/elementwise.cc runtime/executor/activation.cc
runtime/executor/normalization.cc runtime/executor/loss.cc runtime/executor/optimizer.cc
runtime/executor/attention.cc runtime/executor/backend.cc runtime/executor/cpu_backend.cc
runtime/executor/metal_backend_stub.cc runtime/pipeline/dataset.cc runtime/pipeline/batch_pipeline.cc
runtime/storage/durable_io.cc runtime/verifier/plan_validator.cc runtime/storage/checkpoint.cc
runtime/loader/contract.cc runtime/loader/plan_loader.cc runtime/gating/gate.cc
runtime/profiler/runtime_screen.cc runtime/dispatcher/update_engine.cc"

objs=""
list=""
for f in $PAR $SIR $TOK $UPD $RT; do
  o="$OUT/obj/$(echo "$f" | tr '/' '_').o"
  objs="$objs $o"
  list="$list $f"
done
# Compile in parallel, skipping up-to-date objects.
for f in $list; do
  o="$OUT/obj/$(echo "$f" | tr '/' '_').o"
  if [ ! -f "$o" ] || [ "$REF/$f" -nt "$o" ]; then
    echo "$f $o"
  fi
done | xargs -P "$(nproc)" -n 2 sh -c "$CXX $CXXFLAGS -c $REF/\$0 -o \$1"

$CXX $CXXFLAGS "$REF/tool/seeml_update_compile.cc" $objs -o "$OUT/seeml-update-compile"
$CXX $CXXFLAGS "$REF/tool/seeml_plan_probe.cc" $objs -o "$OUT/seeml-plan-probe"
$CXX $CXXFLAGS "$REF/tool/seeml_seeu_dump.cc" $objs -o "$OUT/seeml-seeu-dump"
echo "built: $OUT/seeml-update-compile $OUT/seeml-plan-probe $OUT/seeml-seeu-dump"
