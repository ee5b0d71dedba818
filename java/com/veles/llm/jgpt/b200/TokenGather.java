package com.veles.llm.jgpt.b200;

import static com.veles.llm.jgpt.b200.B200Status.check;
import static java.lang.foreign.ValueLayout.JAVA_BYTE;
import static java.lang.foreign.ValueLayout.JAVA_INT;
import static java.lang.foreign.ValueLayout.JAVA_LONG;

import java.lang.foreign.Arena;
import java.lang.foreign.MemorySegment;

/**
 * All-gather of each GPU's sampled token ids (one JVM thread and one {@link B200Context} per GPU of one box, or one
 * process per GPU).  The sequences are sharded over the GPUs and never interact; this is the only exchange.  The
 * collective runs inside the library (NCCL over NVLink) on a stream of its own; a result is read up to {@code depth}
 * steps after it was submitted, and every wait on the other ranks is bounded ({@link B200Status.GatherTimeoutException}).
 * The reference has no counterpart (it drives device 0 only).
 */
public final class TokenGather implements AutoCloseable {
    private long handle;
    private final int world, maxWords;

    /** Rank 0 creates the 128-byte id and hands it to the other ranks (a file, a socket, the launcher's store). */
    public static byte[] uniqueId() {
        try (Arena a = Arena.ofConfined()) {
            MemorySegment id = a.allocate(128);
            check(JgptB200.commUniqueId(id, 128));
            return id.toArray(JAVA_BYTE);
        }
    }

    public TokenGather(B200Context ctx, byte[] uniqueId, int world, int rank, int maxWords, int depth, int timeoutMs) {
        this.world = world;
        this.maxWords = maxWords;
        try (Arena a = Arena.ofConfined()) {
            MemorySegment id = uniqueId == null ? MemorySegment.NULL : a.allocateFrom(JAVA_BYTE, uniqueId);
            MemorySegment out = a.allocate(JAVA_LONG);
            check(JgptB200.commCreate(ctx.handle(), id, world, rank, maxWords, depth, timeoutMs, out));
            handle = out.get(JAVA_LONG, 0);
        }
    }

    /** This step's words, e.g. (request id, token) pairs; returns at once. */
    public void submit(int[] words) {
        try (Arena a = Arena.ofConfined()) {
            check(JgptB200.commSubmit(handle, a.allocateFrom(JAVA_INT, words), words.length));
        }
    }

    /** True when a result has to be read before the next submit. */
    public boolean mustPop() {
        try (Arena a = Arena.ofConfined()) {
            MemorySegment n = a.allocate(JAVA_INT), m = a.allocate(JAVA_INT);
            check(JgptB200.commInFlight(handle, n, m));
            return m.get(JAVA_INT, 0) != 0;
        }
    }

    /** Oldest step in flight: row r holds rank r's words (length counts[r]); identical on every rank. */
    public int[][] pop(int timeoutMs) {
        try (Arena a = Arena.ofConfined()) {
            MemorySegment words = a.allocate(JAVA_INT, (long) world * maxWords), counts = a.allocate(JAVA_INT, world);
            check(JgptB200.commPop(handle, words, counts, timeoutMs));
            int[][] out = new int[world][];
            for (int r = 0; r < world; r++)
                out[r] = words.asSlice(4L * r * maxWords, 4L * counts.getAtIndex(JAVA_INT, r)).toArray(JAVA_INT);
            return out;
        }
    }

    @Override
    public void close() {
        if (handle != 0) {
            JgptB200.commDestroy(handle);
            handle = 0;
        }
    }
}
