"""Host name and NIC / IPv4 discovery (reference: necklace/utils/osutils.py:32-70)."""
from __future__ import annotations

import socket


def get_hostname() -> str:
    return socket.gethostname()


def get_nic_ip_map() -> dict[str, str]:
    """NIC name -> first IPv4 address."""
    out = {}
    try:
        import psutil
        for nic, addrs in psutil.net_if_addrs().items():
            for a in addrs:
                if a.family == socket.AF_INET:
                    out.setdefault(nic, a.address)
    except Exception:  # noqa: BLE001
        pass
    return out


def get_ip_by_nic(nic: str) -> str | None:
    return get_nic_ip_map().get(nic)


def get_ip_by_prefix(prefix: str) -> str | None:
    for ip in get_nic_ip_map().values():
        if ip.startswith(prefix):
            return ip
    return None


def get_ip_by_first(skip_loopback: bool = True) -> str:
    for ip in get_nic_ip_map().values():
        if not (skip_loopback and ip.startswith("127.")):
            return ip
    return "127.0.0.1"
