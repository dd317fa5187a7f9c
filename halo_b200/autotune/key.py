"""Profile and operator keys (src/autotune/profile_key.cpp:15-47, src/autotune/cpu_ops.cpp:68, src/runtime/profile.cpp:142-172)."""
from __future__ import annotations

import hashlib
import platform
from dataclasses import dataclass, fields

HALO_B200_VERSION = "halo-b200-0.1"

# field name -> must match exactly (True) or version-tolerant (False); order is the reference's
KEY_FIELDS: tuple[tuple[str, bool], ...] = (
    ("halo_version", False), ("model_hash", True), ("pack_id", True), ("gpu_device", True), ("gpu_arch", True),
    ("driver_version", False), ("rocm_version", False), ("vulkan_version", False), ("kernel_version", False), ("os", False),
    ("power_mode", True), ("isa_target", True))


@dataclass(frozen=True)
class ProfileKey:
    halo_version: str = HALO_B200_VERSION
    model_hash: str = ""
    pack_id: str = ""
    gpu_device: str = ""
    gpu_arch: str = ""
    driver_version: str = ""
    rocm_version: str = ""
    vulkan_version: str = ""
    kernel_version: str = ""
    os: str = ""
    power_mode: str = ""
    isa_target: str = ""

    def validate(self) -> None:
        """power_mode = "<platform>|<perf_level>/<power_profile>"; a GPU key with an unknown part is refused
        (src/autotune/profile_key.cpp:37-47, src/profiling/hw_state.cpp:36-58)."""
        pm = self.power_mode
        plat, bar, rest = pm.partition("|")
        if not bar:
            raise ValueError(f"profile key: malformed power mode {pm!r}")
        if plat in ("", "unknown"):
            raise ValueError(f"profile key: platform power mode unknown in {pm!r}")
        if self.gpu_device:
            level, slash, prof = rest.partition("/")
            if not slash or level in ("", "unknown") or prof in ("", "unknown"):
                raise ValueError(f"profile key: GPU power state unknown in {pm!r} for a GPU key")
        for name, must in KEY_FIELDS:
            if must and name not in ("gpu_device", "gpu_arch") and getattr(self, name) == "":
                raise ValueError(f"profile key: {name} is empty")

    def differences(self, other: "ProfileKey") -> int | None:
        """None if a must-match field differs, else the number of version-tolerant fields that differ."""
        n = 0
        for name, must in KEY_FIELDS:
            if getattr(self, name) != getattr(other, name):
                if must:
                    return None
                n += 1
        return n


@dataclass(frozen=True)
class OpKey:
    family: str  # "MATMUL"
    shape: str   # "T=1,K=5120,N=17408,w=q4_k"

    @staticmethod
    def matmul(t_bucket: str | int, cols: int, rows: int, wname: str) -> "OpKey":
        return OpKey("MATMUL", f"T={t_bucket},K={cols},N={rows},w={wname}")


# decode / verify batch buckets (ADR-001 5.6)
T_BUCKETS: tuple[tuple[str, int, int], ...] = (("1", 1, 1), ("2-4", 2, 4), ("5-8", 5, 8), ("9-16", 9, 16))


def pack_id(trunk_hash: str, mtp_hash: str | None = None) -> str:
    """sha256("halo.pack/1\\ntrunk=<h>\\nmtp=<h|none>\\n") (src/runtime/profile.cpp:142-144)."""
    return hashlib.sha256(f"halo.pack/1\ntrunk={trunk_hash}\nmtp={mtp_hash or 'none'}\n".encode()).hexdigest()


def b200_profile_key(info, model_spec: str, *, host_label: str = "b200-hgx", clock_policy: str = "default-clocks",
                     power_cap_w: int = 1000) -> ProfileKey:
    """The key of one B200: gpu_arch = isa_target = sm_100a, gpu_device = PCI vendor:device, driver_version = NVIDIA
    driver + CUDA runtime, rocm / vulkan empty.  With no GGUF file the model hash is the SHA-256 of the synthetic-tensor
    specification string.  `info` is a capi.DeviceInfo."""
    mh = hashlib.sha256(model_spec.encode()).hexdigest()
    arch = info.arch.decode() if isinstance(info.arch, bytes) else str(info.arch)
    pci = info.pci_id.decode() if isinstance(info.pci_id, bytes) else str(info.pci_id)
    key = ProfileKey(model_hash=mh, pack_id=pack_id(mh), gpu_device=pci, gpu_arch=arch,
                     driver_version=f"nvidia-{info.driver_version}/cuda-rt-{info.runtime_version}", kernel_version=platform.release(),
                     os=platform.system().lower(), power_mode=f"{host_label}|{clock_policy}/{power_cap_w}W", isa_target=arch)
    key.validate()
    return key


def key_field_names() -> list[str]:
    return [f.name for f in fields(ProfileKey)]
