#!/usr/bin/env bash
# Replays the reference's own benchmark sweeps with the reference's own programs, built unchanged
# against this library by `make -C oracle reftests` (oracle/_ref/tests):
#   * apps/bench_attention (apps/bench_attention/bench_attention.cu:130-212): seq 512..16384 x
#     head_dim 32/64/128 x causal, cpu / naive / flash / flash_fp16, CSV on stdout;
#   * the strong-scaling job (scripts/slurm/strong_scaling.sbatch: seq 20160, 4 heads, causal
#     zig-zag ring-overlap) and the weak-scaling job (scripts/slurm/weak_scaling.sbatch: 4096 tokens
#     per rank) of ring_attention_cli, launched with the bundled mpirun (minimpi) at every
#     cp_size the box has GPUs for, in the reference's default fp32 and in fp16.
# usage: oracle/replay_reference_sweeps.sh OUT_DIR [ITERS]
set -u
here="$(cd "$(dirname "$0")" && pwd)"
bin="${here}/_ref/tests"
out="${1:?output directory}"
iters="${2:-10}"
mkdir -p "${out}"
export NCCL_NVLS_ENABLE=0 MINIMPI_TIMEOUT_S=300
gpus="$(nvidia-smi -L 2>/dev/null | wc -l)"
header="mode,cp_size,batch,heads,seq,head_dim,causal,zigzag_n,striped,iters,comm_ms,comp_ms,wait_ms,total_ms,max_err"

"${bin}/bench_attention" > "${out}/bench_attention.csv" 2> "${out}/bench_attention.err" || echo "bench_attention failed"

for dtype in fp32 fp16; do
  for kind in strong weak; do
    csv="${out}/${kind}_scaling_${dtype}.csv"
    echo "${header}" > "${csv}"
    for cp in 1 2 4 8; do
      [ "${cp}" -le "${gpus}" ] || continue
      for d in 32 64 128 256; do
        if [ "${kind}" = strong ]; then seq=20160; else seq=$((4096 * cp)); fi
        [ $((seq % (2 * cp))) -eq 0 ] || continue
        "${bin}/mpirun" -n "${cp}" "${bin}/ring_attention_cli" --batch 1 --heads 4 --seq "${seq}" \
          --head_dim "${d}" --causal 1 --mode ring-overlap --zigzag-n 1 --dtype "${dtype}" \
          --iters "${iters}" --csv 2>/dev/null | grep "^ring-overlap," >> "${csv}"
      done
    done
  done
done
# the CLI's mode comparison (scripts/slurm/bench_all.sbatch style) on the widest ring the box allows
csv="${out}/modes_fp16.csv"
echo "${header}" > "${csv}"
cp="${gpus}"; [ "${cp}" -gt 8 ] && cp=8
if [ "${cp}" -ge 2 ]; then
  for mode in allgather ring-blocking ring-overlap; do
    zz="--zigzag-n 1"; [ "${mode}" = allgather ] && zz=""
    "${bin}/mpirun" -n "${cp}" "${bin}/ring_attention_cli" --batch 1 --heads 8 --seq 32768 --head_dim 64 \
      --causal 1 --mode "${mode}" ${zz} --dtype fp16 --iters "${iters}" --csv 2>/dev/null \
      | grep "^${mode}," >> "${csv}"
  done
fi
ls -la "${out}"
