-- Prompt store and roll-out job queue for the RL worker node.
CREATE TABLE IF NOT EXISTS prompts (
    id          BIGSERIAL PRIMARY KEY,
    dataset     TEXT        NOT NULL,
    prompt      TEXT        NOT NULL,
    metadata    JSONB       NOT NULL DEFAULT '{}'::jsonb,
    created_at  TIMESTAMPTZ NOT NULL DEFAULT now()
);
CREATE INDEX IF NOT EXISTS prompts_dataset_idx ON prompts (dataset);

CREATE TABLE IF NOT EXISTS rollout_jobs (
    id          BIGSERIAL PRIMARY KEY,
    prompt_id   BIGINT      NOT NULL REFERENCES prompts (id),
    policy_step BIGINT      NOT NULL,
    status      TEXT        NOT NULL DEFAULT 'pending',
    response    TEXT,
    reward      DOUBLE PRECISION,
    updated_at  TIMESTAMPTZ NOT NULL DEFAULT now()
);
CREATE INDEX IF NOT EXISTS rollout_jobs_status_idx ON rollout_jobs (status, policy_step);
