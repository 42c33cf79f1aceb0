"""Prompt sources for the RL worker node (reference rl/worker_node/prompt_loader.py:15-98).

``DatabasePromptLoader`` reads its connection settings and the SQL that fetches a
prompt from a YAML file in the reference's format (``configs/data_source.example.yaml``):

    database:      {host, dbname, user, password, [port, sslmode, connect_timeout, ...]}
    prompt_query:  SELECT ... LIMIT 1

Every key of ``database`` goes into the connection string as it is.  A sampled
prompt is the first row of the query as a dict keyed by column name, or ``None``
when the query returns nothing.  ``psycopg`` is imported when a connection is
first needed; a connection factory can be injected for tests.
"""
from __future__ import annotations

from pathlib import Path
from typing import Any

import yaml

DEFAULT_CONFIG_PATH = Path(__file__).resolve().parents[2] / "configs" / "data_source.yaml"
_REQUIRED_DB_KEYS = ("host", "dbname", "user", "password")


class PromptLoader:
    """Interface of a prompt source: ``samplePrompt()`` returns one prompt as a dict, or ``None``."""

    def samplePrompt(self) -> dict[str, Any] | None:
        return None


def read_data_source(config_path) -> dict[str, Any]:
    """Load and check a data-source file; returns ``{"database": {...}, "prompt_query": "..."}``."""
    path = Path(config_path)
    if not path.is_file():
        raise FileNotFoundError(f"data source config not found: {path} (copy configs/data_source.example.yaml to "
                                "configs/data_source.yaml and fill in the credentials)")
    with path.open(encoding="utf-8") as handle:
        config = yaml.safe_load(handle)
    if not isinstance(config, dict):
        raise TypeError(f"invalid data source config: {path}")
    database = config.get("database")
    if not isinstance(database, dict):
        raise TypeError("the config must hold a 'database' mapping")
    missing = [key for key in _REQUIRED_DB_KEYS if key not in database]
    if missing:
        raise ValueError(f"'database' is missing required keys: {missing}")
    query = config.get("prompt_query")
    if not isinstance(query, str) or not query.strip():
        raise ValueError("the config must hold a non-empty 'prompt_query' SQL string")
    return config


class DatabasePromptLoader(PromptLoader):
    """Prompts from a PostgreSQL database; one lazily opened, autocommitting connection that is reopened if it
    was closed under us."""

    def __init__(self, config_path=DEFAULT_CONFIG_PATH, connect=None):
        self._config = read_data_source(config_path)
        self._conninfo = self._build_conninfo(self._config["database"])
        self._prompt_query = self._config["prompt_query"]
        self._connect = connect
        self._conn = None

    _load_config = staticmethod(read_data_source)

    @staticmethod
    def _build_conninfo(db_config: dict[str, Any]) -> str:
        return " ".join(f"{key}={value}" for key, value in db_config.items())

    def _get_connection(self):
        if self._conn is None or getattr(self._conn, "closed", False):
            if self._connect is None:
                import psycopg
                from psycopg.rows import dict_row
                self._conn = psycopg.connect(self._conninfo, autocommit=True, row_factory=dict_row)
            else:
                self._conn = self._connect(self._conninfo)
        return self._conn

    def samplePrompt(self) -> dict[str, Any] | None:
        with self._get_connection().cursor() as cursor:
            cursor.execute(self._prompt_query)
            row = cursor.fetchone()
        return None if row is None else dict(row)

    def close(self) -> None:
        if self._conn is not None and not getattr(self._conn, "closed", False):
            self._conn.close()
        self._conn = None

    def __enter__(self):
        return self

    def __exit__(self, *exc) -> None:
        self.close()
