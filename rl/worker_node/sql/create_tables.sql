-- Tables of the RL worker node: the prompt store that DatabasePromptLoader reads, and the roll-out jobs that
-- workers lease from it (one roll-out per prompt, run and policy version).

CREATE TABLE IF NOT EXISTS prompts (
    id           bigint  PRIMARY KEY,
    prompt_text  text    NOT NULL,
    priority     integer NOT NULL DEFAULT 0        -- higher is served first
);

CREATE TABLE IF NOT EXISTS rollout_jobs (
    id                bigserial   PRIMARY KEY,
    run_id            uuid        NOT NULL,
    prompt_id         bigint      NOT NULL REFERENCES prompts (id),
    policy_version    text        NOT NULL,
    status            text        NOT NULL CHECK (status IN ('leased', 'completed', 'failed')),
    worker_id         text        NOT NULL,
    sampled_at        timestamptz NOT NULL DEFAULT now(),
    lease_expires_at  timestamptz NOT NULL,
    completed_at      timestamptz,
    UNIQUE (run_id, policy_version, prompt_id)
);

-- expired leases are found by status and expiry time
CREATE INDEX IF NOT EXISTS rollout_jobs_lease_idx ON rollout_jobs (status, lease_expires_at);
