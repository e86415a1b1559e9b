"""Host / device capability checks (reference: python/llm/src/ipex_llm/utils/isa_checker.py:21-87 checks AVX-512 /
AMX for its CPU kernels).  Here the host library needs only AVX2-class code paths compiled by g++ for the build host,
and the device library needs compute capability 10.0."""
from __future__ import annotations

import platform


class ISAChecker:
    def __init__(self):
        self.flags = set()
        try:
            import cpuinfo
            self.flags = set(cpuinfo.get_cpu_info().get("flags", []))
        except Exception:  # noqa: BLE001
            try:
                with open("/proc/cpuinfo") as f:
                    for line in f:
                        if line.startswith("flags"):
                            self.flags = set(line.split(":", 1)[1].split())
                            break
            except OSError:
                pass

    def check_avx(self):
        return "avx" in self.flags

    def check_avx2(self):
        return "avx2" in self.flags

    def check_avx_vnni(self):
        return "avx_vnni" in self.flags or "avx512_vnni" in self.flags

    def check_avx512(self):
        return "avx512f" in self.flags

    def check_avx512_vnni(self):
        return "avx512_vnni" in self.flags


isa_checker = ISAChecker()


def check_avx_vnni():
    return isa_checker.check_avx_vnni()


def check_avx2():
    return isa_checker.check_avx2()


def check_avx512():
    return isa_checker.check_avx512()


def check_avx512_vnni():
    return isa_checker.check_avx512_vnni()


def is_server():
    return isa_checker.check_avx512()


def is_spr():
    return "amx_tile" in isa_checker.flags


def check_blackwell(device=0) -> bool:
    """True when ``device`` can run the sm_100a kernels of this package."""
    import torch
    if not torch.cuda.is_available():
        return False
    major, _ = torch.cuda.get_device_capability(device)
    return major == 10


def glibc_version():
    return platform.libc_ver()[1]
