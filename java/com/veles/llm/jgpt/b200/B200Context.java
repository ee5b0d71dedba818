package com.veles.llm.jgpt.b200;

import static com.veles.llm.jgpt.b200.B200Status.check;
import static java.lang.foreign.ValueLayout.ADDRESS;
import static java.lang.foreign.ValueLayout.JAVA_INT;
import static java.lang.foreign.ValueLayout.JAVA_LONG;

import java.lang.foreign.Arena;
import java.lang.foreign.MemorySegment;

/**
 * One GPU and one stream: the counterpart of the reference's process-global stream and its
 * {@code TensorOpsGPU.initGPU / isGpuAvailable / requireCuda / synchronizeStream} (TensorOpsGPU.java:87-132,
 * 1197-1203).  Not thread-safe, like the reference's model and cache: one inference thread per context.
 */
public final class B200Context implements AutoCloseable {
    private long handle;
    private final int device;

    public B200Context(int device) {
        try (Arena a = Arena.ofConfined()) {
            MemorySegment out = a.allocate(JAVA_LONG);
            check(JgptB200.ctxCreate(device, out)); // IllegalStateException when no usable GPU (requireCuda)
            handle = out.get(JAVA_LONG, 0);
        }
        this.device = device;
    }

    private static B200Context shared;

    /** The process-wide context on device 0: what the reference's hard-coded device and global stream amount to. */
    public static synchronized B200Context shared() {
        if (shared == null || shared.handle == 0) shared = new B200Context(0);
        return shared;
    }

    public static int deviceCount() {
        try (Arena a = Arena.ofConfined()) {
            MemorySegment out = a.allocate(JAVA_INT);
            check(JgptB200.deviceCount(out));
            return out.get(JAVA_INT, 0);
        }
    }

    /** {@code TensorOpsGPU.isGpuAvailable()}: true when the library opens and sees a device. */
    public static boolean isGpuAvailable() {
        try {
            return deviceCount() > 0;
        } catch (UnsatisfiedLinkError | RuntimeException e) {
            return false;
        }
    }

    public long handle() {
        if (handle == 0) throw new IllegalStateException("context is closed");
        return handle;
    }

    public int device() {
        return device;
    }

    /** {@code TensorOpsGPU.synchronizeStream()}; throws if a kernel recorded a failed self-check. */
    public void synchronize() {
        check(JgptB200.sync(handle()));
    }

    /** {free, total} bytes of the device ({@code getGpuMemoryAllocated0 / Reserved0}). */
    public long[] memInfo() {
        try (Arena a = Arena.ofConfined()) {
            MemorySegment f = a.allocate(JAVA_LONG), t = a.allocate(JAVA_LONG);
            check(JgptB200.memInfo(handle(), f, t));
            return new long[] {f.get(JAVA_LONG, 0), t.get(JAVA_LONG, 0)};
        }
    }

    /** {@code GpuFloatBuffer.allocate}: a raw device allocation, returned as its address. */
    public long devAlloc(long bytes) {
        try (Arena a = Arena.ofConfined()) {
            MemorySegment out = a.allocate(ADDRESS);
            check(JgptB200.devAlloc(handle(), bytes, out)); // OutOfMemoryError like GpuFloatBuffer.allocate
            return out.get(ADDRESS, 0).address();
        }
    }

    public void devFree(long dev) {
        check(JgptB200.devFree(handle(), MemorySegment.ofAddress(dev)));
    }

    /** {@code GpuFloatBuffer.copyTo}: synchronises before returning. */
    public void copyToHost(float[] dst, long dev, int nFloats) {
        try (Arena a = Arena.ofConfined()) {
            MemorySegment h = a.allocate(4L * nFloats, 16);
            check(JgptB200.d2h(handle(), h, MemorySegment.ofAddress(dev), 4L * nFloats));
            MemorySegment.copy(h, java.lang.foreign.ValueLayout.JAVA_FLOAT, 0, dst, 0, nFloats);
        }
    }

    @Override
    public void close() {
        if (handle != 0) {
            JgptB200.ctxDestroy(handle);
            handle = 0;
        }
    }
}
