package com.veles.llm.jgpt.b200;

/**
 * The settings of the B200 KV path, in the reference's style: a {@code JGPT_*} environment variable first, then the
 * matching {@code -Djgpt.*} property, unparsable or out-of-range values ignored (TensorOpsGpuInit.java:30-101,
 * training/LLMConfig.java:190-199).
 *
 * <pre>
 *   JGPT_KV_BACKEND      / jgpt.kv.backend        b200 (default) | anything else = keep the reference's own KV path
 *   JGPT_KV_BLOCK_TOKENS / jgpt.kv.block.tokens   16 (the only size the kernels are built for)
 *   JGPT_KV_POOL_BLOCKS  / jgpt.kv.pool.blocks    blocks of the shared pool; unset = one full context per sequence
 *   JGPT_MAX_SEQ_LEN                              positive override of the configured context
 *   JGPT_RMSNORM_EPS     / jgpt.rmsnorm.eps       (0, 1e-2]; default 1e-5 with JGPT_FP16_MATMUL, else 1e-6
 *   JGPT_B200_LIB        / jgpt.b200.lib          path of libjgpt_b200.so (see {@link B200Library})
 * </pre>
 */
public record B200Config(boolean backendB200, int kvBlockTokens, int kvPoolBlocks, int maxSeqLenOverride, float rmsNormEps) {

    private static String setting(String env, String prop) {
        try {
            String e = System.getenv(env);
            if (e != null && !e.isBlank()) return e.trim();
            if (prop != null) {
                String p = System.getProperty(prop);
                if (p != null && !p.isBlank()) return p.trim();
            }
        } catch (SecurityException ignored) {
            // fall through to the default
        }
        return null;
    }

    private static int positiveInt(String env, String prop, int dflt) {
        String s = setting(env, prop);
        if (s == null) return dflt;
        try {
            int v = Integer.parseInt(s);
            return v > 0 ? v : dflt;
        } catch (NumberFormatException e) {
            return dflt;
        }
    }

    public static B200Config fromEnvironment() {
        String backend = setting("JGPT_KV_BACKEND", "jgpt.kv.backend");
        String fp16 = setting("JGPT_FP16_MATMUL", "jgpt.fp16.matmul");
        boolean fp16On = fp16 != null && (fp16.equals("1") || fp16.equalsIgnoreCase("true"));
        float eps = fp16On ? 1e-5f : 1e-6f;
        String e = setting("JGPT_RMSNORM_EPS", "jgpt.rmsnorm.eps");
        if (e != null) {
            try {
                float v = Float.parseFloat(e);
                if (v > 0f && Float.isFinite(v) && v <= 1e-2f) eps = v;
            } catch (NumberFormatException ignored) {
                // keep the default
            }
        }
        return new B200Config(backend == null || backend.equalsIgnoreCase("b200"), positiveInt("JGPT_KV_BLOCK_TOKENS", "jgpt.kv.block.tokens", 16),
                positiveInt("JGPT_KV_POOL_BLOCKS", "jgpt.kv.pool.blocks", 0), positiveInt("JGPT_MAX_SEQ_LEN", null, 0), eps);
    }

    /** Blocks of a pool for {@code sequences} concurrent sequences of up to {@code maxSeqLen} tokens, unless set explicitly. */
    public int poolBlocksFor(int sequences, int maxSeqLen) {
        return kvPoolBlocks > 0 ? kvPoolBlocks : sequences * ((maxSeqLen + kvBlockTokens - 1) / kvBlockTokens);
    }
}
