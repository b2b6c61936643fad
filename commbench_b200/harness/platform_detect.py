"""What this machine offers to the framework: GPUs (name, compute capability, driver, count),
the CUDA toolchain, NVLink / NVSwitch connectivity, multicast support and whether an RDMA NIC
(InfiniBand / RoCE / EFA) plus ``libibverbs`` is present for the optional verbs transport.

Counterpart of the reference's ``run_eval/platform_detect.py`` (``GPUInfo`` / ``NetworkInfo`` /
``PlatformInfo`` at :14-103, NVIDIA probing through ``nvcc`` and ``nvidia-smi`` at :158-202,
ibverbs / EFA / IB probing at :217-297, the platform string at :372-390, the ``--json`` /
``--quiet`` CLI at :393-434).  This framework targets one vendor and one architecture, so the
AMD branch is not reproduced; instead the record carries what the B200 code paths depend on
(sm_100 check, NVLink peer matrix summary, multicast attribute).

Every probe is a bounded subprocess or a file read; nothing here touches GPU settings.
"""
from __future__ import annotations

import argparse
import json
import os
import platform as _platform
import re
import shutil
import subprocess
import sys
from dataclasses import asdict, dataclass, field


@dataclass
class GpuInfo:
    count: int = 0
    names: list[str] = field(default_factory=list)
    compute_caps: list[str] = field(default_factory=list)
    driver_version: str | None = None
    memory_mib: list[int] = field(default_factory=list)
    nvcc: str | None = None
    nvcc_version: str | None = None
    nvlink_peers: int | None = None          # GPUs reachable over NVLink from GPU 0
    nvswitch: bool | None = None
    multicast: bool | None = None            # CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED on GPU 0

    @property
    def available(self) -> bool:
        return self.count > 0

    @property
    def is_blackwell_dc(self) -> bool:
        """True when every GPU reports compute capability 10.x (B200 / GB200 class)."""
        return bool(self.compute_caps) and all(c.startswith("10.") for c in self.compute_caps)


@dataclass
class NetworkInfo:
    kind: str = "none"                       # "ib", "roce", "efa" or "none"
    devices: list[str] = field(default_factory=list)
    details: dict[str, dict] = field(default_factory=dict)
    has_ibverbs_header: bool = False
    has_ibverbs_lib: bool = False

    @property
    def available(self) -> bool:
        return self.kind != "none" and bool(self.devices)


@dataclass
class PlatformInfo:
    gpu: GpuInfo
    network: NetworkInfo
    hostname: str = ""
    kernel: str = ""

    def platform_string(self) -> str:
        """``B200_NVLINK``, ``NV_IB``, ``NV``, ``CPU`` ...: GPU part then interconnect part."""
        if not self.gpu.available:
            left = "CPU"
        elif self.gpu.is_blackwell_dc:
            left = "B200" if any("B200" in n for n in self.gpu.names) else "SM100"
        else:
            left = "NV"
        parts = [left]
        if self.gpu.available and (self.gpu.nvlink_peers or 0) > 0:
            parts.append("NVLINK")
        if self.network.available:
            parts.append(self.network.kind.upper())
        return "_".join(parts)

    def to_dict(self) -> dict:
        d = asdict(self)
        d["platform"] = self.platform_string()
        d["gpu"]["available"] = self.gpu.available
        d["gpu"]["is_blackwell_dc"] = self.gpu.is_blackwell_dc
        d["network"]["available"] = self.network.available
        return d

    def summary(self) -> str:
        g, n = self.gpu, self.network
        lines = [f"host {self.hostname}  kernel {self.kernel}  platform {self.platform_string()}"]
        if g.available:
            lines.append(f"GPUs: {g.count} x {g.names[0] if g.names else '?'}  "
                         f"cc {','.join(sorted(set(g.compute_caps)))}  driver {g.driver_version}")
            lines.append(f"  nvcc: {g.nvcc or 'not found'} {g.nvcc_version or ''}")
            lines.append(f"  NVLink peers of GPU0: {g.nvlink_peers}  NVSwitch: {g.nvswitch}  "
                         f"multicast: {g.multicast}")
        else:
            lines.append("GPUs: none visible")
        if n.available:
            lines.append(f"RDMA: {n.kind} devices {', '.join(n.devices)}")
        else:
            lines.append("RDMA: no device")
        lines.append(f"  libibverbs header: {n.has_ibverbs_header}  library: {n.has_ibverbs_lib}")
        return "\n".join(lines)


def _run(cmd: list[str], timeout: float = 10.0, runner=None):
    """(ok, stdout).  ``runner`` replaces subprocess for tests."""
    if runner is not None:
        return runner(cmd)
    try:
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout)
        return r.returncode == 0, r.stdout
    except Exception:
        return False, ""


def detect_gpu(runner=None, which=shutil.which) -> GpuInfo:
    info = GpuInfo()
    nvcc = which("nvcc") or ("/usr/local/cuda/bin/nvcc" if os.path.exists("/usr/local/cuda/bin/nvcc")
                             else None)
    if nvcc:
        info.nvcc = nvcc
        ok, out = _run([nvcc, "--version"], runner=runner)
        m = re.search(r"release\s+([\d.]+)", out) if ok else None
        info.nvcc_version = m.group(1) if m else None
    smi = which("nvidia-smi")
    if not smi:
        return info
    ok, out = _run([smi, "--query-gpu=name,driver_version,compute_cap,memory.total",
                    "--format=csv,noheader,nounits"], runner=runner)
    if not ok:
        return info
    for line in out.strip().splitlines():
        f = [x.strip() for x in line.split(",")]
        if len(f) < 3:
            continue
        info.names.append(f[0])
        info.driver_version = f[1]
        info.compute_caps.append(f[2])
        try:
            info.memory_mib.append(int(float(f[3])))
        except (IndexError, ValueError):
            pass
    info.count = len(info.names)
    if info.count > 1:
        ok, out = _run([smi, "topo", "-m"], runner=runner)
        if ok:
            info.nvlink_peers, info.nvswitch = parse_topology(out)
    elif info.count == 1:
        info.nvlink_peers, info.nvswitch = 0, False
    return info


def parse_topology(text: str) -> tuple[int, bool | None]:
    """From ``nvidia-smi topo -m``: how many GPUs GPU0 reaches over NVLink (``NV<k>`` cells), and
    whether every pair has the same link count (the signature of an NVSwitch fabric)."""
    # Matrix rows start with "GPUn" at column 0 (the header row is indented) and hold an "X".
    rows = [ln.split() for ln in text.splitlines() if re.match(r"^GPU\d+\s", ln) and " X " in f" {ln} ".replace("\t", " ")]
    if not rows:
        return 0, None
    n = len(rows)
    cells0 = rows[0][1:1 + n]
    peers = sum(1 for c in cells0 if re.fullmatch(r"NV\d+", c))
    counts = set()
    for r in rows:
        for c in r[1:1 + n]:
            m = re.fullmatch(r"NV(\d+)", c)
            if m:
                counts.add(int(m.group(1)))
    switch = (peers == n - 1 and len(counts) == 1) if n > 2 else (None if peers == 0 else False)
    if n == 2 and peers == 1:
        switch = None       # two GPUs cannot tell a switch from a direct bridge
    return peers, switch


def detect_multicast() -> bool | None:
    """Multicast (NVLS) attribute of device 0 through the native library, when it is built and a
    GPU is present; ``None`` otherwise."""
    try:
        import torch

        if not torch.cuda.is_available():
            return None
        from .. import _native

        return _native.load().cb_symm_multicast_supported(0) > 0
    except Exception:
        return None


def detect_network(runner=None, which=shutil.which, sysfs: str = "/sys/class/infiniband",
                   include_dirs=("/usr/include", "/usr/local/include")) -> NetworkInfo:
    net = NetworkInfo()
    net.has_ibverbs_header = any(os.path.exists(os.path.join(d, "infiniband", "verbs.h"))
                                 for d in include_dirs)
    for d in ("/usr/lib/x86_64-linux-gnu", "/usr/lib64", "/usr/lib", "/usr/local/lib",
              "/usr/lib/aarch64-linux-gnu"):
        try:
            if any(f.startswith("libibverbs.so") for f in os.listdir(d)):
                net.has_ibverbs_lib = True
                break
        except OSError:
            continue
    fi = which("fi_info")
    if fi:
        ok, out = _run([fi, "-p", "efa"], runner=runner)
        if ok and "provider: efa" in out:
            devs = sorted(set(re.findall(r"domain:\s*(\S+)", out)))
            net.kind, net.devices = "efa", devs
            for dv in devs:
                net.details[dv] = {"type": "EFA"}
            return net
    devs: list[str] = []
    if os.path.isdir(sysfs):
        devs = sorted(os.listdir(sysfs))
    elif which("ibv_devices"):
        ok, out = _run([which("ibv_devices")], runner=runner)
        if ok:
            devs = [ln.split()[0] for ln in out.splitlines()[2:] if ln.strip()]
    if not devs:
        return net
    net.devices = devs
    kinds = set()
    for dv in devs:
        layer = None
        try:
            with open(os.path.join(sysfs, dv, "ports", "1", "link_layer")) as f:
                layer = f.read().strip()
        except OSError:
            pass
        k = "roce" if layer == "Ethernet" else "ib"
        kinds.add(k)
        net.details[dv] = {"type": k.upper(), "link_layer": layer}
    net.kind = "ib" if "ib" in kinds else "roce"
    return net


def detect_platform(runner=None, which=shutil.which) -> PlatformInfo:
    gpu = detect_gpu(runner, which)
    if gpu.available and runner is None:
        gpu.multicast = detect_multicast()
    return PlatformInfo(gpu=gpu, network=detect_network(runner, which),
                        hostname=_platform.node(), kernel=_platform.release())


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="Detect GPUs, NVLink fabric and RDMA NICs")
    ap.add_argument("--json", action="store_true")
    ap.add_argument("--quiet", action="store_true", help="print only the platform string")
    a = ap.parse_args(argv)
    info = detect_platform()
    if a.json:
        print(json.dumps(info.to_dict(), indent=1))
    elif a.quiet:
        print(info.platform_string())
    else:
        print(info.summary())
    return 0


if __name__ == "__main__":
    sys.exit(main())
