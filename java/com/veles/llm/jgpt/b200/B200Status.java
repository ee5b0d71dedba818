package com.veles.llm.jgpt.b200;

import java.lang.foreign.MemorySegment;

/**
 * Status codes of the C ABI and their mapping to the exception classes the reference throws for the same
 * misuse (model/GptKvForward.java:47-60, 131-141; model/KvCacheGpu.java:18-75; GpuFloatBuffer.java:127-130).
 */
public final class B200Status {
    private B200Status() {}

    public static final int OK = 0, INVALID_ARGUMENT = 1, ILLEGAL_STATE = 2, OUT_OF_RANGE = 3, OUT_OF_MEMORY = 4,
            POOL_EXHAUSTED = 5, BAD_HANDLE = 6, CUDA = 7, UNSUPPORTED = 8, DEVICE_CHECK = 9, IO = 10, NCCL = 11, TIMEOUT = 12;

    /** Raised for KV-pool exhaustion: the paged store has no free block or sequence slot (no reference counterpart). */
    public static final class PoolExhaustedException extends IllegalStateException {
        public PoolExhaustedException(String m) {
            super(m);
        }
    }

    /** A bounded wait on another rank ran out; the step stays in flight and may be read again. */
    public static final class GatherTimeoutException extends RuntimeException {
        public GatherTimeoutException(String m) {
            super(m);
        }
    }

    public static String lastError() {
        MemorySegment p = JgptB200.lastError();
        return p.equals(MemorySegment.NULL) ? "" : p.reinterpret(4096).getString(0);
    }

    /** Throws what the reference would throw; returns normally on {@link #OK}. */
    public static void check(int rc) {
        if (rc == OK) return;
        String msg = lastError();
        switch (rc) {
            case INVALID_ARGUMENT -> throw new IllegalArgumentException(msg);
            case ILLEGAL_STATE, UNSUPPORTED, DEVICE_CHECK, BAD_HANDLE, CUDA, NCCL -> throw new IllegalStateException(msg);
            case OUT_OF_RANGE -> throw new IndexOutOfBoundsException(msg);
            case OUT_OF_MEMORY -> throw new OutOfMemoryError(msg);
            case POOL_EXHAUSTED -> throw new PoolExhaustedException(msg);
            case IO -> throw new java.io.UncheckedIOException(new java.io.IOException(msg));
            case TIMEOUT -> throw new GatherTimeoutException(msg);
            default -> throw new IllegalStateException("jgpt_b200 status " + rc + ": " + msg);
        }
    }
}
