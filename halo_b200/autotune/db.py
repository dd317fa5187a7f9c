"""The persistent profile database: SQLite, schema v1 of the reference (src/autotune/db.cpp:55-111).

Same eight tables and column names, `PRAGMA application_id = 0x48414C4F`, `schema_version(app='halo.profile',
version=1)`, WAL journal, foreign keys on, `quick_check` at open, writes in one IMMEDIATE transaction with bound
parameters only, UPSERT of the winner on (hardware, model, operator, backend), UTC timestamps `YYYY-MM-DDTHH:MM:SSZ`
(include/halo/autotune/db.h:1-22).  A symlinked file, a foreign SQLite file, a newer schema and a corrupt file are
refused with a typed error (include/halo/autotune/db.h:44-52; cases of tests/unit/autotune/test_db.cpp:175-319).
"""
from __future__ import annotations

import json
import os
import sqlite3
import time
from dataclasses import asdict
from pathlib import Path

from .candidate import Candidate
from .key import KEY_FIELDS, OpKey, ProfileKey

APPLICATION_ID = 0x48414C4F
APP_NAME = "halo.profile"
SCHEMA_VERSION = 1
WINNER_METRIC = "median_ns"

_HW_COLS = ("halo_version", "gpu_device", "gpu_arch", "driver_version", "rocm_version", "vulkan_version", "kernel_version", "os",
            "power_mode", "isa_target")

_SCHEMA = """
CREATE TABLE schema_version(id INTEGER PRIMARY KEY CHECK (id = 1), app TEXT NOT NULL, version INTEGER NOT NULL);
CREATE TABLE hardware_profile(id INTEGER PRIMARY KEY,
  halo_version TEXT NOT NULL, gpu_device TEXT NOT NULL, gpu_arch TEXT NOT NULL, driver_version TEXT NOT NULL,
  rocm_version TEXT NOT NULL, vulkan_version TEXT NOT NULL, kernel_version TEXT NOT NULL, os TEXT NOT NULL,
  power_mode TEXT NOT NULL, isa_target TEXT NOT NULL, created_at TEXT NOT NULL,
  UNIQUE(halo_version, gpu_device, gpu_arch, driver_version, rocm_version, vulkan_version, kernel_version, os, power_mode, isa_target));
CREATE TABLE tier_bandwidth(id INTEGER PRIMARY KEY,
  hardware_profile_id INTEGER NOT NULL REFERENCES hardware_profile(id) ON DELETE CASCADE,
  tier TEXT NOT NULL, processor TEXT NOT NULL, label TEXT NOT NULL, threads INTEGER NOT NULL, buffer_bytes INTEGER NOT NULL,
  read_gbps REAL NOT NULL, write_gbps REAL NOT NULL, copy_gbps REAL NOT NULL, stats_json TEXT NOT NULL, measured_at TEXT NOT NULL);
CREATE TABLE model_profile(id INTEGER PRIMARY KEY, model_hash TEXT NOT NULL, pack_id TEXT NOT NULL, created_at TEXT NOT NULL,
  UNIQUE(model_hash, pack_id));
CREATE TABLE operator_profile(id INTEGER PRIMARY KEY, family TEXT NOT NULL, shape TEXT NOT NULL, UNIQUE(family, shape));
CREATE TABLE kernel_candidate(id INTEGER PRIMARY KEY,
  operator_profile_id INTEGER NOT NULL REFERENCES operator_profile(id) ON DELETE CASCADE,
  backend TEXT NOT NULL, params TEXT NOT NULL, UNIQUE(operator_profile_id, backend, params));
CREATE TABLE benchmark_run(id INTEGER PRIMARY KEY,
  kind TEXT NOT NULL CHECK (kind IN ('tune', 'baseline', 'bench')),
  hardware_profile_id INTEGER REFERENCES hardware_profile(id), model_profile_id INTEGER REFERENCES model_profile(id),
  kernel_candidate_id INTEGER REFERENCES kernel_candidate(id),
  engine TEXT NOT NULL, backend TEXT NOT NULL, pack TEXT NOT NULL, context INTEGER NOT NULL, mode TEXT NOT NULL,
  power_mode TEXT NOT NULL, strategy TEXT, stability TEXT, median REAL, rejected TEXT, stats_json TEXT, record_json TEXT,
  created_at TEXT NOT NULL);
CREATE INDEX benchmark_run_latest ON benchmark_run(kind, backend, pack, context, mode, created_at);
CREATE TABLE winning_configuration(id INTEGER PRIMARY KEY,
  hardware_profile_id INTEGER NOT NULL REFERENCES hardware_profile(id),
  model_profile_id INTEGER NOT NULL REFERENCES model_profile(id),
  operator_profile_id INTEGER NOT NULL REFERENCES operator_profile(id),
  backend TEXT NOT NULL, kernel_candidate_id INTEGER NOT NULL REFERENCES kernel_candidate(id),
  benchmark_run_id INTEGER REFERENCES benchmark_run(id),
  strategy TEXT NOT NULL, metric TEXT NOT NULL, value REAL NOT NULL, created_at TEXT NOT NULL,
  UNIQUE(hardware_profile_id, model_profile_id, operator_profile_id, backend));
"""
TABLES = ("benchmark_run", "hardware_profile", "kernel_candidate", "model_profile", "operator_profile", "schema_version",
          "tier_bandwidth", "winning_configuration")


class DbError(RuntimeError):
    """kind: Corrupt | NotHaloDb | ForeignVersion | Busy | Io | Constraint | Internal (include/halo/autotune/db.h:44-52)."""

    def __init__(self, kind: str, message: str):
        self.kind = kind
        super().__init__(f"profile db ({kind}): {message}")


def utc_now() -> str:
    return time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime())


class ProfileDb:
    def __init__(self, path: str | os.PathLike, *, readonly: bool = False, create: bool = True):
        self.path = Path(path)
        self.readonly = readonly
        if self.path.is_symlink():
            raise DbError("Io", f"{self.path} is a symbolic link")  # src/autotune/sqlite.cpp:104-107
        exists = self.path.exists()
        if not exists and (readonly or not create):
            raise DbError("Io", f"{self.path} does not exist")
        try:
            uri = f"file:{self.path}?mode={'ro' if readonly else 'rwc'}"
            self.conn = sqlite3.connect(uri, uri=True, isolation_level=None, timeout=5.0)
            self.conn.execute("PRAGMA foreign_keys = ON")
            fresh = not exists or self.path.stat().st_size == 0
            if fresh:
                self._create()
            else:
                self._verify()
            if not readonly:
                self.conn.execute("PRAGMA journal_mode = WAL")
        except sqlite3.DatabaseError as e:
            raise DbError("Corrupt" if "malformed" in str(e) or "not a database" in str(e) else "Io", str(e)) from e

    def close(self) -> None:
        self.conn.close()

    def _create(self) -> None:
        c = self.conn
        c.execute(f"PRAGMA application_id = {APPLICATION_ID}")
        c.execute("BEGIN IMMEDIATE")
        for stmt in [s.strip() for s in _SCHEMA.split(";") if s.strip()]:
            c.execute(stmt)
        c.execute("INSERT INTO schema_version(id, app, version) VALUES (1, ?, ?)", (APP_NAME, SCHEMA_VERSION))
        c.execute("COMMIT")

    def _verify(self) -> None:
        c = self.conn
        if c.execute("PRAGMA quick_check").fetchone()[0] != "ok":
            raise DbError("Corrupt", f"{self.path} fails quick_check")
        if c.execute("PRAGMA application_id").fetchone()[0] != APPLICATION_ID:
            raise DbError("NotHaloDb", f"{self.path} is not a HALO profile database (application id)")
        try:
            row = c.execute("SELECT app, version FROM schema_version WHERE id = 1").fetchone()
        except sqlite3.OperationalError as e:
            raise DbError("NotHaloDb", f"{self.path} has no schema_version table") from e
        if row is None or row[0] != APP_NAME:
            raise DbError("NotHaloDb", f"{self.path} was not written by HALO")
        if row[1] > SCHEMA_VERSION:
            raise DbError("ForeignVersion", f"{self.path} has schema version {row[1]}, this build reads up to {SCHEMA_VERSION}")
        have = {r[0] for r in c.execute("SELECT name FROM sqlite_master WHERE type = 'table'")}
        missing = set(TABLES) - have
        if missing:
            raise DbError("Corrupt", f"{self.path} lacks tables {sorted(missing)}")

    # ---- ensure_* helpers (run inside the caller's transaction) ---------------------------------------------------
    def _require_writable(self) -> None:
        if self.readonly:
            raise DbError("Io", "database opened read-only")

    def _ensure_hardware(self, key: ProfileKey) -> int:
        vals = tuple(getattr(key, c) for c in _HW_COLS)
        where = " AND ".join(f"{c} = ?" for i, c in enumerate(_HW_COLS))
        row = self.conn.execute(f"SELECT id FROM hardware_profile WHERE {where}", vals).fetchone()
        if row:
            return row[0]
        cols = ", ".join(_HW_COLS)
        marks = ", ".join("?" for _ in range(len(_HW_COLS) + 1))
        return self.conn.execute(f"INSERT INTO hardware_profile({cols}, created_at) VALUES ({marks})", vals + (utc_now(),)).lastrowid

    def _ensure_model(self, key: ProfileKey) -> int:
        row = self.conn.execute("SELECT id FROM model_profile WHERE model_hash = ? AND pack_id = ?", (key.model_hash, key.pack_id)).fetchone()
        if row:
            return row[0]
        return self.conn.execute("INSERT INTO model_profile(model_hash, pack_id, created_at) VALUES (?, ?, ?)",
                                 (key.model_hash, key.pack_id, utc_now())).lastrowid

    def _ensure_operator(self, op: OpKey) -> int:
        row = self.conn.execute("SELECT id FROM operator_profile WHERE family = ? AND shape = ?", (op.family, op.shape)).fetchone()
        if row:
            return row[0]
        return self.conn.execute("INSERT INTO operator_profile(family, shape) VALUES (?, ?)", (op.family, op.shape)).lastrowid

    def _ensure_candidate(self, op_id: int, backend: str, params: str) -> int:
        row = self.conn.execute("SELECT id FROM kernel_candidate WHERE operator_profile_id = ? AND backend = ? AND params = ?",
                                (op_id, backend, params)).fetchone()
        if row:
            return row[0]
        return self.conn.execute("INSERT INTO kernel_candidate(operator_profile_id, backend, params) VALUES (?, ?, ?)",
                                 (op_id, backend, params)).lastrowid

    # ---- writes ----------------------------------------------------------------------------------------------------------
    def persist_tune(self, key: ProfileKey, result) -> bool:
        """One IMMEDIATE transaction: every measured candidate becomes a benchmark_run row of kind 'tune', the winner (if
        any) is upserted into winning_configuration (src/autotune/db.cpp:353-403).  Returns whether a winner was written;
        with no winner an existing winner stays."""
        self._require_writable()
        key.validate()
        c = self.conn
        try:
            c.execute("BEGIN IMMEDIATE")
            hw, model, op = self._ensure_hardware(key), self._ensure_model(key), self._ensure_operator(result.key)
            now = utc_now()
            winner_text = result.winner.to_string() if result.winner is not None else None
            winner_run = winner_cand = None
            for cr in result.candidates:
                params = cr.candidate.to_string()
                cand = self._ensure_candidate(op, result.backend, params)
                if not cr.measured:
                    continue
                run = c.execute(
                    "INSERT INTO benchmark_run(kind, hardware_profile_id, model_profile_id, kernel_candidate_id, engine, backend, pack, "
                    "context, mode, power_mode, strategy, stability, median, rejected, stats_json, record_json, created_at) "
                    "VALUES ('tune', ?, ?, ?, 'halo', ?, ?, 0, ?, ?, ?, ?, ?, ?, ?, ?, ?)",
                    (hw, model, cand, result.backend, key.pack_id, f"{result.key.family}/{result.key.shape}", key.power_mode, result.strategy,
                     cr.stability, cr.stats.get("median"), cr.rejected, json.dumps(cr.stats), json.dumps(cr.to_json()), now)).lastrowid
                if winner_text is not None and params == winner_text:
                    winner_run, winner_cand = run, cand
            wrote = False
            if winner_text is not None:
                if winner_cand is None:
                    raise DbError("Constraint", f"persist_tune: winner {winner_text} is not a measured candidate of the result")
                c.execute(
                    "INSERT INTO winning_configuration(hardware_profile_id, model_profile_id, operator_profile_id, kernel_candidate_id, "
                    "benchmark_run_id, strategy, metric, value, created_at, backend) VALUES (?,?,?,?,?,?,?,?,?,?) "
                    "ON CONFLICT(hardware_profile_id, model_profile_id, operator_profile_id, backend) DO UPDATE SET "
                    "kernel_candidate_id = excluded.kernel_candidate_id, benchmark_run_id = excluded.benchmark_run_id, "
                    "strategy = excluded.strategy, metric = excluded.metric, value = excluded.value, created_at = excluded.created_at",
                    (hw, model, op, winner_cand, winner_run, result.strategy, WINNER_METRIC, result.winner_median_ns, now, result.backend))
                wrote = True
            c.execute("COMMIT")
            return wrote
        except sqlite3.OperationalError as e:
            self._rollback()
            raise DbError("Busy" if "locked" in str(e) or "busy" in str(e) else "Internal", str(e)) from e
        except Exception:
            self._rollback()
            raise

    def _rollback(self) -> None:
        try:
            self.conn.execute("ROLLBACK")
        except sqlite3.Error:
            pass

    def record_tier_bandwidth(self, key: ProfileKey, *, tier: str, processor: str, label: str, threads: int, buffer_bytes: int,
                              read_gbps: float, write_gbps: float, copy_gbps: float, stats: dict | None = None) -> None:
        """A measured bandwidth under the key (the tuner records one before tuning, tools/halo/tune.cpp:302-316)."""
        self._require_writable()
        c = self.conn
        c.execute("BEGIN IMMEDIATE")
        try:
            hw = self._ensure_hardware(key)
            c.execute("INSERT INTO tier_bandwidth(hardware_profile_id, tier, processor, label, threads, buffer_bytes, read_gbps, write_gbps, "
                      "copy_gbps, stats_json, measured_at) VALUES (?,?,?,?,?,?,?,?,?,?,?)",
                      (hw, tier, processor, label, threads, buffer_bytes, read_gbps, write_gbps, copy_gbps, json.dumps(stats or {}), utc_now()))
            c.execute("COMMIT")
        except Exception:
            self._rollback()
            raise

    # ---- reads -----------------------------------------------------------------------------------------------------------
    def winners(self, op: OpKey, backend: str) -> list[tuple[ProfileKey, Candidate, float, str]]:
        """Every stored winner of (operator, backend label) with the key it was tuned under: (key, candidate, median ns,
        created_at).  Winners are kept per backend label, so "cuda" rows coexist with "cpu" rows."""
        rows = self.conn.execute(
            "SELECT h.halo_version, m.model_hash, m.pack_id, h.gpu_device, h.gpu_arch, h.driver_version, h.rocm_version, h.vulkan_version, "
            "h.kernel_version, h.os, h.power_mode, h.isa_target, k.params, w.value, w.created_at "
            "FROM winning_configuration w JOIN hardware_profile h ON h.id = w.hardware_profile_id "
            "JOIN model_profile m ON m.id = w.model_profile_id JOIN operator_profile o ON o.id = w.operator_profile_id "
            "JOIN kernel_candidate k ON k.id = w.kernel_candidate_id "
            "WHERE o.family = ? AND o.shape = ? AND w.backend = ? ORDER BY w.id", (op.family, op.shape, backend)).fetchall()
        names = [n for n, _ in KEY_FIELDS]
        return [(ProfileKey(**dict(zip(names, r[:12]))), Candidate.parse(r[12]), float(r[13]), r[14]) for r in rows]

    def counts(self) -> dict[str, int]:
        return {t: self.conn.execute(f"SELECT COUNT(*) FROM {t}").fetchone()[0] for t in TABLES}


def key_as_dict(key: ProfileKey) -> dict:
    return asdict(key)
