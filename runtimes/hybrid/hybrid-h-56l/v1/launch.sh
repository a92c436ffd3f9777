#!/bin/sh
# Entry point of this recipe version.  The model identity and the tuning come only from the reviewed files beside this script
# (profile.json, model.lock.json); the operator's site file names the model folder and the port.
#   ./launch.sh [VERB] [--site site.json] [--profile NAME] [--state-dir DIR] [--crc] [--no-wait]
# Verbs: doctor install-deps setup print-command start status stop logs verify diagnostics reset-state   (default: start)
set -eu
here=$(cd "$(dirname "$0")" && pwd -P)
repo=$(cd "$here/../../../.." && pwd -P)
verb=start
case "${1-}" in
  -h|--help|help) sed -n '2,5p' "$0"; exit 0 ;;
  doctor|install-deps|setup|print-command|start|status|stop|logs|verify|diagnostics|reset-state) verb=$1; shift ;;
  --*|"") ;;
  *) printf 'Unknown command: %s\n' "$1" >&2; exit 2 ;;
esac
if [ "$verb" = start ] && [ "$(id -u)" = 0 ] && [ -z "${REXL3_ALLOW_ROOT-}" ]; then
  printf '%s\n' 'RUN_AS_NORMAL_USER: start without sudo (set REXL3_ALLOW_ROOT=1 inside a container)' >&2
  exit 2
fi
cd "$repo"
exec "${PYTHON:-python3}" -m rexl3_b200.launcher "$verb" --recipe "$here" "$@"
