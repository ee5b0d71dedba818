package com.veles.llm.jgpt.b200;

import java.lang.foreign.Arena;
import java.lang.foreign.SymbolLookup;
import java.nio.file.Files;
import java.nio.file.Path;

/**
 * Finds and opens {@code libjgpt_b200.so}, in the order the reference looks for its own native library
 * (cuda/TensorCudaLibrary.java:42-101): the system property first, then the environment variable, then paths
 * relative to the working directory, then the platform's library path.
 *
 * <pre>
 *   -Djgpt.b200.lib=/abs/path/libjgpt_b200.so
 *   JGPT_B200_LIB=/abs/path/libjgpt_b200.so
 *   build/libjgpt_b200.so, jgpt_b200/lib/libjgpt_b200.so, ./libjgpt_b200.so
 *   java.library.path / LD_LIBRARY_PATH  (libjgpt_b200.so)
 * </pre>
 *
 * The library has no CPU fallback; if it cannot be opened the error is an {@link UnsatisfiedLinkError}, like the
 * reference's loader.  The lookup lives as long as the JVM (global arena): handles bound from it stay valid.
 */
public final class B200Library {
    private B200Library() {}

    private static volatile SymbolLookup lookup;
    private static volatile String loadedFrom;

    public static String loadedFrom() {
        return loadedFrom;
    }

    public static SymbolLookup lookup() {
        SymbolLookup l = lookup;
        if (l != null) return l;
        synchronized (B200Library.class) {
            if (lookup == null) lookup = open();
            return lookup;
        }
    }

    private static SymbolLookup open() {
        String prop = System.getProperty("jgpt.b200.lib");
        if (prop != null && !prop.isBlank()) return openFile(Path.of(prop.trim()), "jgpt.b200.lib");
        String env = System.getenv("JGPT_B200_LIB");
        if (env != null && !env.isBlank()) return openFile(Path.of(env.trim()), "JGPT_B200_LIB");
        for (String rel : new String[] {"build/libjgpt_b200.so", "jgpt_b200/lib/libjgpt_b200.so", "libjgpt_b200.so"}) {
            Path p = Path.of(rel).normalize();
            if (Files.isRegularFile(p)) return openFile(p, rel);
        }
        try {
            SymbolLookup l = SymbolLookup.libraryLookup(System.mapLibraryName("jgpt_b200"), Arena.global());
            loadedFrom = "libjgpt_b200.so (library path)";
            return l;
        } catch (IllegalArgumentException e) {
            throw new UnsatisfiedLinkError(
                    "libjgpt_b200.so not found: set -Djgpt.b200.lib or JGPT_B200_LIB, or put it on the library path ("
                            + e.getMessage() + ")");
        }
    }

    private static SymbolLookup openFile(Path p, String how) {
        if (!Files.isRegularFile(p)) throw new UnsatisfiedLinkError(how + " not found: " + p);
        SymbolLookup l = SymbolLookup.libraryLookup(p.toAbsolutePath(), Arena.global());
        loadedFrom = p.toAbsolutePath().toString();
        return l;
    }
}
