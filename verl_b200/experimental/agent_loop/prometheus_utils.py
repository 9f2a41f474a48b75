"""Point a Prometheus instance at the rollout servers (verl/experimental/agent_loop/prometheus_utils.py:28-111).

Writes ``config.file`` with one scrape job over the servers' ``/metrics`` endpoints and asks the local Prometheus
(``config.port``) to reload. One box, so no per-node fan-out."""

from __future__ import annotations

import logging
import os
import urllib.request

import yaml

logger = logging.getLogger(__name__)


def update_prometheus_config(config, server_addresses: list[str], rollout_name: str | None = None, reload: bool = True) -> bool:
    if not server_addresses:
        logger.warning("No server addresses available to update Prometheus config")
        return False
    get = config.get if hasattr(config, "get") else lambda k, d=None: getattr(config, k, d)
    doc = {"global": {"scrape_interval": "10s", "evaluation_interval": "10s"},
           "scrape_configs": [{"job_name": "rollout", "static_configs": [{"targets": list(server_addresses)}]}]}
    path = get("file")
    try:
        os.makedirs(os.path.dirname(path), exist_ok=True)
        with open(path, "w") as f:
            yaml.dump(doc, f, default_flow_style=False, indent=2)
    except OSError as e:
        logger.error("Failed to update Prometheus configuration: %s", e)
        return False
    print(f"Updated Prometheus configuration at {path} with {len(server_addresses)} {(rollout_name or 'rollout').upper()} servers")
    if reload:
        try:
            req = urllib.request.Request(f"http://127.0.0.1:{get('port', 9090)}/-/reload", method="POST")
            urllib.request.urlopen(req, timeout=2).read()
        except Exception as e:  # no Prometheus running is not an error for training
            logger.info("Prometheus reload skipped: %s", e)
    return True
