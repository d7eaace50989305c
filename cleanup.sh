#!/usr/bin/env bash
# Remove shared-memory segments left by a crashed CPU-tier run (counterpart of backend/test/cleanup.sh).
# Processes are not touched: stop your own job by its pid.
rm -f /dev/shm/stb200-shm-meta-* /dev/shm/stb200-shm-data-* /tmp/stellatrain-b200-controller-*.pid
