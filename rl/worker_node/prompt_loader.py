"""Sample prompts from a Postgres table (reference rl/worker_node/prompt_loader.py:23-98).

Connection settings come from a YAML file (see ``configs/data_source.example.yaml``).
``psycopg`` is imported when a connection is first needed; a connection factory can
be injected for tests.
"""
from __future__ import annotations

from pathlib import Path

import yaml


class DatabasePromptLoader:
    REQUIRED = ("host", "port", "dbname", "user")

    def __init__(self, config_path, connect=None):
        with Path(config_path).open(encoding="utf-8") as handle:
            config = yaml.safe_load(handle) or {}
        source = config.get("data_source") or {}
        missing = [k for k in self.REQUIRED if k not in source]
        if missing:
            raise ValueError(f"data_source is missing keys: {missing}")
        self.source = source
        self.table = source.get("table", "prompts")
        self.dataset = source.get("dataset")
        if not self.table.replace("_", "").isalnum():
            raise ValueError("table name must be alphanumeric")
        self._connect = connect
        self._connection = None

    def _conn(self):
        if self._connection is None:
            if self._connect is None:
                import psycopg
                self._connect = psycopg.connect
            keys = ("host", "port", "dbname", "user", "password")
            self._connection = self._connect(**{k: self.source[k] for k in keys if k in self.source})
        return self._connection

    def samplePrompt(self):
        """One random row as ``{"id", "prompt", "metadata"}`` or ``None`` if the table is empty."""
        query = f"SELECT id, prompt, metadata FROM {self.table}"
        params = ()
        if self.dataset:
            query += " WHERE dataset = %s"
            params = (self.dataset,)
        query += " ORDER BY random() LIMIT 1"
        with self._conn().cursor() as cursor:
            cursor.execute(query, params)
            row = cursor.fetchone()
        if row is None:
            return None
        return {"id": row[0], "prompt": row[1], "metadata": row[2]}

    def close(self):
        if self._connection is not None:
            self._connection.close()
            self._connection = None
