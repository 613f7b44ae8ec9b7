import java.io.IOException;
import java.io.PrintWriter;
import java.lang.foreign.Arena;
import java.lang.foreign.MemorySegment;
import java.lang.foreign.ValueLayout;
import java.nio.ByteOrder;
import java.nio.channels.FileChannel;
import java.nio.file.Path;
import java.nio.file.StandardOpenOption;

import org.beehive.jitllm.backend.cpu.InferenceCore;
import org.beehive.jitllm.inference.state.LlamaState;
import org.beehive.jitllm.inference.state.State;
import org.beehive.jitllm.inference.weights.standard.LlamaStandardWeights;
import org.beehive.jitllm.model.llama.LlamaConfiguration;
import org.beehive.jitllm.runtime.tensor.DataType;
import org.beehive.jitllm.tensor.standard.FP32FloatTensor;
import org.beehive.jitllm.tensor.standard.FloatTensor;
import org.beehive.jitllm.tensor.standard.Q4_0FloatTensor;
import org.beehive.jitllm.tensor.standard.Q4_KFloatTensor;
import org.beehive.jitllm.tensor.standard.Q8_0FloatTensor;

/**
 * Cross-check of the C oracle against jitLLM's own CPU path, for a machine that has a JDK.
 *
 * <p>The model is the recipe of LlamaCpuOperationEquivalenceTest (a tiny Llama, teacher-forced
 * tokens, InferenceCore.forwardJava position by position), but with weights in GGUF Q8_0 / Q4_0 /
 * Q4_K blocks. jitLLM has no encoder, so the blocks come from a file written by
 * make_crosscheck_input.py (next to this class): it holds the configuration, the tokens, and every
 * tensor's bytes in the order the constructor of LlamaStandardWeights takes them. This class wraps
 * those bytes in the reference's own Q*FloatTensor classes, runs the forward pass and writes the raw
 * bits of every logit, one line per position; tests/test_oracle_java_crosscheck.py compares that
 * file with the oracle's logits bit for bit.
 *
 * <p>Build and run, from the jitLLM checkout (module path as for its own tests):
 *
 * <pre>
 *   python tests/java/make_crosscheck_input.py Q4_K tests/java/crosscheck_q4_k.bin
 *   javac --add-modules jdk.incubator.vector -cp target/classes -d /tmp/xc QuantizedForwardCrossCheck.java
 *   java  --add-modules jdk.incubator.vector --enable-preview -cp target/classes:/tmp/xc \
 *         QuantizedForwardCrossCheck tests/java/crosscheck_q4_k.bin tests/java/crosscheck_q4_k.logits
 * </pre>
 */
public final class QuantizedForwardCrossCheck {

    private static final ValueLayout.OfInt I32 = ValueLayout.JAVA_INT_UNALIGNED.withOrder(ByteOrder.LITTLE_ENDIAN);
    private static final ValueLayout.OfFloat F32 = ValueLayout.JAVA_FLOAT_UNALIGNED.withOrder(ByteOrder.LITTLE_ENDIAN);

    private final MemorySegment file;
    private long at;

    private QuantizedForwardCrossCheck(MemorySegment file) {
        this.file = file;
    }

    private int nextInt() {
        int v = file.get(I32, at);
        at += 4;
        return v;
    }

    private float nextFloat() {
        float v = file.get(F32, at);
        at += 4;
        return v;
    }

    private MemorySegment nextBytes(long n) {
        at = (at + 31) / 32 * 32; // every tensor starts on a 32-byte boundary
        MemorySegment s = file.asSlice(at, n);
        at += n;
        return s;
    }

    private static long rowBytes(int type, long elements) {
        switch (type) {
            case 8: return elements / 32 * 34; // Q8_0
            case 2: return elements / 32 * 18; // Q4_0
            case 12: return elements / 256 * 144; // Q4_K
            default: throw new IllegalArgumentException("GGML type " + type);
        }
    }

    private FloatTensor quantised(int type, int elements) {
        MemorySegment s = nextBytes(rowBytes(type, elements));
        switch (type) {
            case 8: return new Q8_0FloatTensor(elements, s);
            case 2: return new Q4_0FloatTensor(elements, s);
            default: return new Q4_KFloatTensor(elements, s);
        }
    }

    private FloatTensor plain(int elements) {
        return new FP32FloatTensor(elements, nextBytes(4L * elements));
    }

    public static void main(String[] args) throws IOException {
        if (args.length != 2) {
            System.err.println("usage: QuantizedForwardCrossCheck <input.bin> <output.logits>");
            System.exit(2);
        }
        try (Arena arena = Arena.ofConfined();
                FileChannel ch = FileChannel.open(Path.of(args[0]), StandardOpenOption.READ)) {
            MemorySegment file = ch.map(FileChannel.MapMode.READ_ONLY, 0, ch.size(), arena);
            QuantizedForwardCrossCheck in = new QuantizedForwardCrossCheck(file);
            if (in.nextInt() != 0x43584C4A) { // "JLXC"
                throw new IOException("not a cross-check input file");
            }
            int dim = in.nextInt(), hidden = in.nextInt(), layers = in.nextInt(), heads = in.nextInt();
            int kvHeads = in.nextInt(), vocab = in.nextInt(), context = in.nextInt(), type = in.nextInt();
            int nTokens = in.nextInt();
            float eps = in.nextFloat(), theta = in.nextFloat();
            int[] tokens = new int[nTokens];
            for (int i = 0; i < nTokens; i++) {
                tokens[i] = in.nextInt();
            }
            LlamaConfiguration config =
                    new LlamaConfiguration("Q", dim, hidden, layers, heads, kvHeads, vocab, context, eps, theta);
            int kvDim = config.kvDim();
            int headSize = config.headSize();

            FloatTensor embedding = in.quantised(type, vocab * dim);
            FloatTensor[] attNorm = new FloatTensor[layers], wq = new FloatTensor[layers], wk = new FloatTensor[layers];
            FloatTensor[] wv = new FloatTensor[layers], wo = new FloatTensor[layers], ffnNorm = new FloatTensor[layers];
            FloatTensor[] w1 = new FloatTensor[layers], w2 = new FloatTensor[layers], w3 = new FloatTensor[layers];
            for (int l = 0; l < layers; l++) {
                attNorm[l] = in.plain(dim);
                wq[l] = in.quantised(type, dim * dim);
                wk[l] = in.quantised(type, kvDim * dim);
                wv[l] = in.quantised(type, kvDim * dim);
                wo[l] = in.quantised(type, dim * dim);
                ffnNorm[l] = in.plain(dim);
                w1[l] = in.quantised(type, hidden * dim);
                w2[l] = in.quantised(type, dim * hidden);
                w3[l] = in.quantised(type, hidden * dim);
            }
            FloatTensor finalNorm = in.plain(dim);
            FloatTensor ropeReal = in.plain(context * (headSize / 2));
            FloatTensor ropeImag = in.plain(context * (headSize / 2));
            FloatTensor wcls = in.quantised(type, vocab * dim);
            DataType weightType = type == 8 ? DataType.Q8_0 : (type == 2 ? DataType.Q4_0 : DataType.Q4_K);
            LlamaStandardWeights weights =
                    new LlamaStandardWeights(embedding, attNorm, wq, wk, wv, wo, ffnNorm, w1, w2, w3, finalNorm,
                            ropeReal, ropeImag, wcls, weightType);

            State state = new LlamaState(config, -1);
            try (PrintWriter out = new PrintWriter(args[1])) {
                for (int position = 0; position < nTokens; position++) {
                    FloatTensor logits = InferenceCore.forwardJava(config, weights, state, tokens[position], position);
                    StringBuilder line = new StringBuilder(9 * vocab);
                    for (int i = 0; i < vocab; i++) {
                        line.append(String.format("%08x", Float.floatToRawIntBits(logits.getFloat(i))));
                        line.append(i + 1 < vocab ? ' ' : '\n');
                    }
                    out.print(line);
                }
            }
        }
    }
}
