#!/bin/sh
# Launch the default profile of this recipe version with the site file given as $1.
set -eu
here=$(cd "$(dirname "$0")/../../../.." && pwd)
cd "$here"
exec python -m rexl3_b200.recipes --root runtimes --family hybrid --model gdn-hybrid-27b --version v1 --site "$1" --exec
