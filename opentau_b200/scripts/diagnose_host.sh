#!/usr/bin/env bash
# Read-only snapshot of a training / serving host, written next to benchmark results so that two latency or
# throughput records can be compared knowing what differed between the machines (same role as the reference's
# src/opentau/scripts/diagnose_host.sh).  Nothing is changed on the host: every command only queries.
#
#   bash opentau_b200/scripts/diagnose_host.sh [output_dir]
set -u

out_dir="${1:-benchmark_results}"
mkdir -p "$out_dir"
report="${out_dir}/$(hostname)_host.txt"
py="${BENCH_PYTHON:-python3}"

probe() {           # probe "<title>" <command...>: a failing or missing tool leaves a note, never aborts the report
    local title="$1"; shift
    {
        printf '\n## %s\n$ %s\n' "$title" "$*"
        bash -c "$*" 2>&1 || echo "(unavailable)"
    } >> "$report"
}

{
    echo "# host report"
    echo "host: $(hostname)"
    echo "utc:  $(date -u +%Y-%m-%dT%H:%M:%SZ)"
    echo "kernel: $(uname -srm)"
} > "$report"

probe "GPUs" "nvidia-smi --query-gpu=index,name,driver_version,memory.total,memory.used,pstate,power.draw,power.limit,clocks.sm,clocks.max.sm,clocks.mem,utilization.gpu,pcie.link.gen.current,pcie.link.width.current --format=csv"
probe "GPU clock event reasons" "nvidia-smi --query-gpu=index,clocks_event_reasons.active,clocks_event_reasons.sw_power_cap,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown --format=csv"
probe "GPU topology (NVLink / NVSwitch)" "nvidia-smi topo -m"
probe "NVLink state" "nvidia-smi nvlink --status | head -60"
probe "compute processes on the GPUs" "nvidia-smi --query-compute-apps=gpu_uuid,pid,name,used_memory --format=csv"
probe "CPU" "lscpu | grep -E 'Model name|^CPU\\(s\\)|Thread|Socket|NUMA|MHz'"
probe "CPU governor" "cat /sys/devices/system/cpu/cpu0/cpufreq/scaling_governor"
probe "memory" "free -h"
probe "block devices" "lsblk -d -o NAME,ROTA,SIZE,MODEL | grep -v loop"
probe "shared memory and temp space" "df -h /dev/shm /tmp"
probe "limits" "ulimit -a | grep -E 'open files|locked memory|max user processes'"
probe "python stack" "$py -c \"import torch, sys; print('python', sys.version.split()[0]); print('torch', torch.__version__, 'cuda', torch.version.cuda, 'nccl', '.'.join(map(str, torch.cuda.nccl.version())) if torch.cuda.is_available() else ''); print('devices', torch.cuda.device_count()); print('capability', torch.cuda.get_device_capability(0) if torch.cuda.is_available() else None)\""
probe "native extensions of this package" "$py -c \"import pathlib, opentau_b200.ops as o; d = pathlib.Path(o.__file__).parent; print(*sorted(p.name for p in d.rglob('*.so')), sep='\\n')\""
probe "environment knobs" "env | grep -E '^(OPENTAU_B200_|NCCL_|CUDA_VISIBLE|PYTORCH_CUDA_ALLOC|OMP_NUM_THREADS)' | sort"
probe "busiest processes" "ps -eo pid,pcpu,pmem,comm --sort=-pcpu | head -8"

echo "report: $report"
