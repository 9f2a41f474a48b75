"""Data re-sharding hooks around a worker computation (verl/workers/sharding_manager/base.py)."""

from __future__ import annotations


class BaseShardingManager:
    def __init__(self):
        self.timing = {}

    def __enter__(self):
        return self

    def __exit__(self, exc_type, exc_value, traceback):
        return False

    def preprocess_data(self, data):
        return data

    def postprocess_data(self, data):
        return data
