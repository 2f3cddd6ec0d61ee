"""NUMA placement of a rank's host threads and pinned memory next to its GPU.

Pinned host buffers that feed a GPU over PCIe should live on the socket the GPU hangs off: a buffer on the
other socket crosses the inter-socket link on every copy, and with eight ranks copying at once that link, not
PCIe, sets the pace. Linux places freshly allocated pages on the node of the CPU that allocates them, so
pinning the process to the GPU's node before it allocates is enough; no libnuma is needed.

The reference keeps its host segment NUMA-local in the allocator itself
(``csrc/kernels/backend/symmetric.hpp`` of the reference: ``ElasticSymmetricMemory`` asks for the device's
host NUMA id) and its tests leave the binding of the process to the launcher
(``tests/legacy/test_low_latency.py:316``).
"""
from __future__ import annotations

import os
from typing import List, Optional, Set


def parse_cpu_list(text: str) -> List[int]:
    """``"0-3,8,10-11"`` -> ``[0, 1, 2, 3, 8, 10, 11]`` (the format of ``/sys/devices/system/node/node*/cpulist``)."""
    cpus: List[int] = []
    for part in text.strip().split(','):
        part = part.strip()
        if not part:
            continue
        if '-' in part:
            lo, hi = part.split('-', 1)
            cpus.extend(range(int(lo), int(hi) + 1))
        else:
            cpus.append(int(part))
    return cpus


def pci_numa_node(pci_bus_id: str, sysfs_root: str = '/sys') -> Optional[int]:
    """NUMA node of a PCI device (``"0000:1b:00.0"``; NVML's eight-digit domain is accepted), ``None`` if unknown."""
    bdf = pci_bus_id.strip().lower()
    if bdf.count(':') == 2 and len(bdf.split(':')[0]) == 8:
        bdf = bdf[4:]
    try:
        with open(os.path.join(sysfs_root, 'bus/pci/devices', bdf, 'numa_node')) as f:
            node = int(f.read().strip())
    except (OSError, ValueError):
        return None
    return node if node >= 0 else None


def node_cpus(node: int, sysfs_root: str = '/sys') -> List[int]:
    try:
        with open(os.path.join(sysfs_root, f'devices/system/node/node{node}/cpulist')) as f:
            return parse_cpu_list(f.read())
    except OSError:
        return []


def gpu_pci_bus_id(device_index: int) -> Optional[str]:
    try:
        import torch
        props = torch.cuda.get_device_properties(device_index)
        return '%04x:%02x:%02x.0' % (props.pci_domain_id, props.pci_bus_id, props.pci_device_id)
    except Exception:
        return None


def gpu_host_numa_id(device_index: int) -> Optional[int]:
    """The driver's answer (``cudaDevAttrHostNumaId``) for systems whose sysfs does not tell."""
    try:
        from cuda.bindings import runtime as cudart
        err, node = cudart.cudaDeviceGetAttribute(cudart.cudaDeviceAttr.cudaDevAttrHostNumaId, device_index)
        return int(node) if int(err) == 0 and int(node) >= 0 else None
    except Exception:
        return None


def bind_to_gpu_node(device_index: int, sysfs_root: str = '/sys') -> Optional[dict]:
    """Restricts the calling process to the CPUs of the NUMA node of GPU ``device_index``.

    Call it before pinned host memory is allocated. Returns ``{'node': n, 'num_cpus': k}``, or ``None`` when the
    node cannot be determined or none of its CPUs is available to the process (nothing is changed then).
    """
    bdf = gpu_pci_bus_id(device_index)
    node = pci_numa_node(bdf, sysfs_root) if bdf is not None else None
    if node is None:
        node = gpu_host_numa_id(device_index)
    if node is None:
        return None
    allowed: Set[int] = set(os.sched_getaffinity(0))
    target = allowed & set(node_cpus(node, sysfs_root))
    if not target:
        return None
    os.sched_setaffinity(0, target)
    return {'node': node, 'num_cpus': len(target)}
