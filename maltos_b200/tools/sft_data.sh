#!/usr/bin/env sh
# Packed SFT shards; first argument or PRESET picks the preset (olmo | custom), the rest are environment variables.
set -eu
cd "$(dirname -- "$0")/../.."
exec python3 -m maltos_b200.tools.data_presets sft "$@"
