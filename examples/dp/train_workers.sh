#!/bin/bash
# Start one scheduler and N workers of train_mnist_dp.py on this host, one GPU each
# (reference: examples/dp/mnist/pytorch/train_workers.sh).
#   ./train_workers.sh 4            # 4 workers on GPUs 0..3
#   NO_CUDA=1 ./train_workers.sh 2  # CPU
set -e
N=${1:-2}
DIR=$(cd "$(dirname "$0")" && pwd)
TMP=$(mktemp -d)
EXTRA=""
[ -n "$NO_CUDA" ] && EXTRA="--no-cuda"
python "$DIR/train_mnist_dp.py" -r scheduler -w "$N" -u "ipc://$TMP/svr.ipc" -e "${EPOCHS:-1}" &
for ((r = 0; r < N; r++)); do
  python "$DIR/train_mnist_dp.py" -r worker -w "$N" -k "$r" -g "$r" -u "ipc://$TMP/w$r.ipc" \
    -s "ipc://$TMP/svr.ipc" -t dp --dataset-len "${DATASET_LEN:-2000}" $EXTRA &
done
wait
