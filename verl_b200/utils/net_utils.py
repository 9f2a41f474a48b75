"""Network helpers (role of verl/utils/net_utils.py)."""

from __future__ import annotations

import ipaddress
import socket


def is_ipv4(ip: str) -> bool:
    try:
        ipaddress.IPv4Address(ip)
        return True
    except ipaddress.AddressValueError:
        return False


def is_ipv6(ip: str) -> bool:
    try:
        ipaddress.IPv6Address(ip)
        return True
    except ipaddress.AddressValueError:
        return False


def is_valid_ipv6_address(ip: str) -> bool:
    return is_ipv6(ip)


def get_free_port(host: str = "127.0.0.1") -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind((host, 0))
        return s.getsockname()[1]


def format_url(host: str, port: int, scheme: str = "http") -> str:
    return f"{scheme}://[{host}]:{port}" if is_ipv6(host) else f"{scheme}://{host}:{port}"
