#!/bin/bash
# Launchers for one 8 x B200 NVSwitch node (counterpart of the reference's PBS script scripts/train_aurora.sh, which
# starts 1,920 ranks on 160 Aurora nodes). One process per GPU through torchrun; the rendezvous uses 127.0.0.1.
#   ./launch_8xb200.sh train [overrides...]       WP = 8 training of the 1.3 B-class model (experiment b200_1p3b_wp8)
#   ./launch_8xb200.sh train-sp [overrides...]    WP 4 x SP 2 (fused Ulysses exchange)
#   ./launch_8xb200.sh train-tp [overrides...]    WP 4 x SP 2 with the MLP weights split over every SP pair (model.TP=2)
#   ./launch_8xb200.sh train-pp [overrides...]    the 13 B-class model as PP 2 x WP 2 x SP 2 (pipeline engine)
#   ./launch_8xb200.sh train-ref [overrides...]   the reference's own `train` experiment (24 blocks, 60 x 60 windows),
#                                                 one replica per GPU (data parallel)
#   ./launch_8xb200.sh infer [args...]            one ensemble member per GPU, device-resident rollout
#   ./launch_8xb200.sh bench                      the flagship training-step benchmark at 1, 2, 4, 8 GPUs
set -euo pipefail
N=${NGPU:-8}
RUN="python -m torch.distributed.run --nnodes=1 --nproc-per-node $N --master-addr 127.0.0.1 --master-port ${PORT:-29500}"
cd "$(dirname "$0")/../.."
mode=${1:-train}; shift || true
case "$mode" in
  train)    exec $RUN -m aeris_gb_b200.cli.train experiment=b200_1p3b_wp8 "$@" ;;
  train-sp) exec $RUN -m aeris_gb_b200.cli.train experiment=b200_1p3b_wp4_sp2 "$@" ;;
  train-tp) exec $RUN -m aeris_gb_b200.cli.train experiment=b200_1p3b_wp4_sp2 model.TP=2 "$@" ;;
  train-pp) exec $RUN -m aeris_gb_b200.cli.train experiment=b200_13b_pp2_wp2_sp2 "$@" ;;
  train-ref) exec $RUN -m aeris_gb_b200.cli.train experiment=train model.SP=1 model.WP_X=1 model.WP_Y=1 model.PP=1 \
               model.chunk_windows=16 data.gas=1 "$@" ;;
  infer)    exec $RUN -m aeris_gb_b200.cli.wp_inference --member-parallel --members "$N" --random-init "$@" ;;
  bench)    python bench.py --gpus 1
            for n in 2 4 8; do
              python -m torch.distributed.run --nnodes=1 --nproc-per-node $n --master-addr 127.0.0.1 --master-port 29500 bench.py --gpus $n
            done ;;
  *) echo "unknown mode $mode" >&2; exit 2 ;;
esac
