package com.veles.llm.jgpt.b200;

import static com.veles.llm.jgpt.b200.B200Status.check;
import static java.lang.foreign.ValueLayout.JAVA_INT;
import static java.lang.foreign.ValueLayout.JAVA_LONG;

import java.lang.foreign.Arena;
import java.lang.foreign.MemorySegment;

/**
 * Continuous batching over one model and one KV pool: requests are admitted first-in first-out as blocks and sequence
 * slots free up (their whole reservation at once), finished sequences are evicted least-recently-used first, every
 * step prefills the newly admitted prompts in one call and advances the running requests by one token in another.
 * The reference generates one sequence per call with a fresh cache (model/GptAutoregressiveGenerator.java:108-206); this
 * is the serving loop around the same forward step.  The policy lives in the library and is deterministic: the same
 * submissions give the same admissions, evictions and block tables.
 */
public final class ContinuousBatcher implements AutoCloseable {
    /** One sampled token of one request in one step. */
    public record Sampled(int request, int token) {}

    /** What a step did: the tokens it sampled, and how many requests are running / waiting afterwards. */
    public record StepResult(Sampled[] sampled, int running, int waiting) {
        public boolean idle() {
            return running == 0 && waiting == 0;
        }
    }

    private long handle;
    private final int maxRunning;

    public ContinuousBatcher(B200Model model, KvPool pool, int maxRunning, int maxRowsPerCall) {
        this.maxRunning = maxRunning;
        try (Arena a = Arena.ofConfined()) {
            MemorySegment out = a.allocate(JAVA_LONG);
            check(JgptB200.schedCreate(model.handle(), pool.handle(), maxRunning, maxRowsPerCall, model.maxSeqLen, out));
            handle = out.get(JAVA_LONG, 0);
        }
    }

    /**
     * Queues a request; returns its id.  IllegalArgumentException when prompt + maxNewTokens - 1 exceeds the context
     * (there is no sliding window while batching) or needs more blocks than the pool has.
     */
    public int submit(int[] prompt, int maxNewTokens) {
        try (Arena a = Arena.ofConfined()) {
            MemorySegment id = a.allocate(JAVA_INT);
            check(JgptB200.schedSubmit(handle, a.allocateFrom(JAVA_INT, prompt), prompt.length, maxNewTokens, id));
            return id.get(JAVA_INT, 0);
        }
    }

    public StepResult step() {
        try (Arena a = Arena.ofConfined()) {
            MemorySegment pairs = a.allocate(JAVA_INT, 2L * maxRunning), n = a.allocate(JAVA_INT), run = a.allocate(JAVA_INT),
                    wait = a.allocate(JAVA_INT);
            check(JgptB200.schedStep(handle, pairs, maxRunning, n, run, wait));
            Sampled[] s = new Sampled[n.get(JAVA_INT, 0)];
            for (int i = 0; i < s.length; i++) s[i] = new Sampled(pairs.getAtIndex(JAVA_INT, 2L * i), pairs.getAtIndex(JAVA_INT, 2L * i + 1));
            return new StepResult(s, run.get(JAVA_INT, 0), wait.get(JAVA_INT, 0));
        }
    }

    /** Tokens sampled so far for a request. */
    public int[] tokens(int request) {
        try (Arena a = Arena.ofConfined()) {
            MemorySegment n = a.allocate(JAVA_INT), state = a.allocate(JAVA_INT), seq = a.allocate(JAVA_INT);
            check(JgptB200.schedResult(handle, request, MemorySegment.NULL, 0, n, state, seq));
            int cnt = n.get(JAVA_INT, 0);
            MemorySegment out = a.allocate(JAVA_INT, Math.max(cnt, 1));
            check(JgptB200.schedResult(handle, request, out, cnt, n, state, seq));
            return out.asSlice(0, 4L * cnt).toArray(JAVA_INT);
        }
    }

    @Override
    public void close() {
        if (handle != 0) {
            JgptB200.schedDestroy(handle);
            handle = 0;
        }
    }
}
