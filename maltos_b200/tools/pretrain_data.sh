#!/usr/bin/env sh
# Token shards of the pre-training subset; every setting is an environment variable (see data_presets.py).
set -eu
cd "$(dirname -- "$0")/../.."
exec python3 -m maltos_b200.tools.data_presets pretrain "$@"
