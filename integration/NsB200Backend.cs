// NOT COMPILED: no .NET SDK exists where this library is built.  tests/test_integration_cs.py checks that every native
// call below names an import of NsB200Native.cs with the right number of arguments and that every abstract member of
// Backend (src/NeuralSharp/Backends/Backend.cs:66-282) is overridden.
//
// Sibling of src/NeuralSharp/Backends/Cuda/CudaBackend.cs: the Backend a Device returns for a B200 (see
// DeviceSelection.md).  It covers the operators of the cached decoder step -- what Tensor dispatch, Linear,
// MultiHeadAttention, DecodingContext, TokenSampler and CharGpt.Generate call (Backend.cs:68-86, 95-129, 140, 172,
// 193-199, 219-281) -- on the library's float32 operator surface, whose entry points keep Backend's argument lists.
// Training, convolution and the other operators outside that path throw NotSupportedException: a model is trained on
// the existing backends and served here.
using System.Runtime.InteropServices;
using static NeuralSharp.Backends.B200.NsB200Native;

namespace NeuralSharp.Backends.B200;

internal sealed class NsB200Storage(NsB200Backend backend, ulong pointer, int length) : Storage(backend, length)
{
    public readonly ulong Pointer = pointer;
}

internal sealed unsafe class NsB200Backend : Backend
{
    private static readonly Dictionary<int, NsB200Backend> Instances = [];

    private readonly nint _device;
    private readonly int _ordinal;

    // Freed blocks, by exact length (the reference's pool has the same shape, CudaBackend.cs:36,185-223).  Return may
    // run on the finalizer thread, so it only touches these dictionaries under the lock and never calls the library.
    private readonly Dictionary<int, Stack<ulong>> _pool = [];
    private Dictionary<int, Stack<ulong>>? _captureFree;
    private long _inUse, _cached;

    public string Name { get; }

    public static int DeviceCount
    {
        get
        {
            return ns_device_count(out int count) == 0 ? count : 0;
        }
    }

    public static NsB200Backend Get(int ordinal)
    {
        lock (Instances)
        {
            if (!Instances.TryGetValue(ordinal, out var backend))
            {
                Instances[ordinal] = backend = new NsB200Backend(ordinal);
            }

            return backend;
        }
    }

    private NsB200Backend(int ordinal)
    {
        _ordinal = ordinal;
        Check(ns_device_open(ordinal, out _device), nameof(ns_device_open));
        byte* name = stackalloc byte[128];
        Check(ns_device_info(_device, name, null, null, null), nameof(ns_device_info));
        Name = Marshal.PtrToStringUTF8((IntPtr)name) ?? $"B200 {ordinal}";
    }

    private static ulong P(Storage storage) => ((NsB200Storage)storage).Pointer;

    private static ulong P(Storage? storage, bool optional) => storage is null ? 0UL : P(storage);

    private static long Bytes(int length) => (long)length * sizeof(float);

    private static NotSupportedException OffPath(string member) =>
        new($"{member} is outside the inference path this backend serves; use the CPU or the CUDA backend for it.");

    // ------------------------------------------------------------------------------------------------ memory

    public override Storage Allocate(int length, bool zeroed)
    {
        ulong pointer = 0;
        lock (_pool)
        {
            if (_pool.TryGetValue(length, out var bucket) && bucket.Count > 0)
            {
                pointer = bucket.Pop();
                _cached -= Bytes(length);
            }

            _inUse += Bytes(length);
        }

        if (pointer == 0)
        {
            int result = ns_alloc(_device, (ulong)Bytes(length), 0, out pointer);
            if (result == ErrMemory)
            {
                // give cached blocks back and try once more, as the reference does on CUDA_ERROR_OUT_OF_MEMORY
                ReleaseCachedMemory();
                result = ns_alloc(_device, (ulong)Bytes(length), 0, out pointer);
            }

            if (result != 0)
            {
                lock (_pool)
                {
                    _inUse -= Bytes(length);
                }

                Check(result, nameof(ns_alloc));
            }
        }

        if (zeroed)
        {
            Check(ns_memset32_async(_device, pointer, 0, (ulong)length), nameof(ns_memset32_async));
        }

        return new NsB200Storage(this, pointer, length);
    }

    public override void Return(Storage storage)
    {
        var s = (NsB200Storage)storage;
        lock (_pool)
        {
            // while a graph is being recorded, freed blocks stay with the graph: it writes to them on every replay
            var target = _captureFree ?? _pool;
            if (!target.TryGetValue(s.Length, out var bucket))
            {
                target[s.Length] = bucket = new Stack<ulong>();
            }

            bucket.Push(s.Pointer);
            _inUse -= Bytes(s.Length);
            _cached += Bytes(s.Length);
        }
    }

    public override MemoryUsage GetMemoryUsage()
    {
        lock (_pool)
        {
            return new MemoryUsage(_inUse, _cached, null);
        }
    }

    public override void ReleaseCachedMemory()
    {
        List<ulong> blocks = [];
        lock (_pool)
        {
            foreach (var (length, bucket) in _pool)
            {
                while (bucket.Count > 0)
                {
                    blocks.Add(bucket.Pop());
                    _cached -= Bytes(length);
                }
            }
        }

        if (blocks.Count == 0)
        {
            return;
        }

        Check(ns_stream_sync(_device), nameof(ns_stream_sync));
        foreach (ulong pointer in blocks)
        {
            Check(ns_free(_device, pointer), nameof(ns_free));
        }
    }

    public override void Upload(ReadOnlySpan<float> source, Storage destination)
    {
        fixed (float* p = source)
        {
            Check(ns_h2d(_device, P(destination), p, (ulong)source.Length * sizeof(float)), nameof(ns_h2d));
        }
    }

    public override void Download(Storage source, Span<float> destination) => DownloadRange(source, 0, destination);

    public override void DownloadRange(Storage source, int offset, Span<float> destination)
    {
        fixed (float* p = destination)
        {
            Check(ns_d2h(_device, p, P(source) + (ulong)offset * sizeof(float), (ulong)destination.Length * sizeof(float)), nameof(ns_d2h));
        }
    }

    public override void Fill(Storage y, int n, float value) =>
        Check(ns_memset32_async(_device, P(y), BitConverter.SingleToUInt32Bits(value), (ulong)n), nameof(ns_memset32_async));

    public override void Copy(Storage x, Storage y, int n) =>
        Check(ns_d2d_async(_device, P(y), P(x), (ulong)n * sizeof(float)), nameof(ns_d2d_async));

    public override void Synchronize() => Check(ns_stream_sync(_device), nameof(ns_stream_sync));

    // ------------------------------------------------------------------------------------------------ element-wise

    public override void Binary(BinaryOp op, Storage a, Storage b, Storage c, int n)
    {
        if (op != BinaryOp.Add)
        {
            throw OffPath($"Binary({op})");   // the decoder's residual connections only add (Layers/Attention.cs:201-205)
        }

        Check(ns_f32_add(_device, P(a), P(b), P(c), n), nameof(ns_f32_add));
    }

    public override void Affine(Storage x, Storage y, int n, float alpha, float beta) =>
        Check(ns_f32_affine(_device, P(x), P(y), n, alpha, beta), nameof(ns_f32_affine));

    public override void AddRowVector(Storage a, Storage v, Storage c, int rows, int cols) =>
        Check(ns_f32_add_row_vector(_device, P(a), P(v), P(c), rows, cols), nameof(ns_f32_add_row_vector));

    public override void AddBroadcastScalar(Storage s, Storage y, int n, float scale) =>
        Check(ns_f32_add_broadcast_scalar(_device, P(s), P(y), n, scale), nameof(ns_f32_add_broadcast_scalar));

    // ------------------------------------------------------------------------------------------------ products and shape operators

    public override void BatchedMatMul(Storage a, Storage b, Storage c, int batch, int m, int n, int k, bool transA, bool transB, float beta) =>
        Check(ns_f32_batched_matmul(_device, P(a), P(b), P(c), batch, m, n, k, transA ? 1 : 0, transB ? 1 : 0, beta), nameof(ns_f32_batched_matmul));

    public override void Softmax(Storage x, Storage y, int rows, int cols, bool log)
    {
        if (log)
        {
            throw OffPath("Softmax(log: true)");
        }

        Check(ns_f32_scale_mask_softmax(_device, P(x), 0, P(y), rows, cols, 1, 1f), nameof(ns_f32_scale_mask_softmax));
    }

    public override void ArgMax(Storage x, Storage y, int rows, int cols) =>
        Check(ns_f32_argmax(_device, P(x), P(y), rows, cols), nameof(ns_f32_argmax));

    public override void Gather(Storage table, Storage indices, Storage y, int count, int dim, int vocabulary) =>
        Check(ns_f32_gather(_device, P(table), P(indices), P(y), count, dim, vocabulary), nameof(ns_f32_gather));

    public override void Permute(Storage x, Storage y, ReadOnlySpan<int> outShape, ReadOnlySpan<int> inStrides, bool accumulate)
    {
        fixed (int* shape = outShape)
        fixed (int* strides = inStrides)
        {
            Check(ns_f32_permute(_device, P(x), P(y), shape, strides, outShape.Length, accumulate ? 1 : 0), nameof(ns_f32_permute));
        }
    }

    public override void Copy2D(Storage src, int srcOffset, int srcStride, Storage dst, int dstOffset, int dstStride, int rows, int cols, bool accumulate) =>
        Check(ns_f32_copy2d(_device, P(src), srcOffset, srcStride, P(dst), dstOffset, dstStride, rows, cols, accumulate ? 1 : 0), nameof(ns_f32_copy2d));

    // ------------------------------------------------------------------------------------------------ fused inference kernels

    public override void ScaleMaskSoftmax(Storage x, Storage? mask, Storage y, int rows, int cols, int maskRows, float scale) =>
        Check(ns_f32_scale_mask_softmax(_device, P(x), P(mask, optional: true), P(y), rows, cols, maskRows, scale), nameof(ns_f32_scale_mask_softmax));

    public override void LayerNormFused(Storage x, Storage gamma, Storage beta, Storage y, int rows, int cols, float eps) =>
        Check(ns_f32_layernorm_fused(_device, P(x), P(gamma), P(beta), P(y), rows, cols, eps), nameof(ns_f32_layernorm_fused));

    public override void BiasGelu(Storage x, Storage bias, Storage y, int n, int cols) =>
        Check(ns_f32_bias_gelu(_device, P(x), P(bias), P(y), n, cols), nameof(ns_f32_bias_gelu));

    // ------------------------------------------------------------------------------------------------ incremental decoding

    public override void DecoderMask(Storage position, Storage mask, int rows, int capacity) =>
        Check(ns_f32_decoder_mask(_device, P(position), P(mask), rows, capacity), nameof(ns_f32_decoder_mask));

    public override void KeyValueWrite(Storage source, Storage cache, Storage position, int heads, int steps, int capacity, int dim) =>
        Check(ns_f32_key_value_write(_device, P(source), P(cache), P(position), heads, steps, capacity, dim), nameof(ns_f32_key_value_write));

    public override void SampleRows(Storage logits, Storage ids, Storage stats, Storage step, int rows, int vocabulary,
        int rowStride, int rowOffset, float temperature, int topK, float topP, float minP, uint seed) =>
        Check(ns_f32_sample_rows(_device, P(logits), P(ids), P(stats), P(step), rows, vocabulary, rowStride, rowOffset, temperature, topK, topP, minP, seed),
            nameof(ns_f32_sample_rows));

    public override void PenalizeRows(Storage logits, Storage work, Storage history, Storage length, int rows, int vocabulary,
        int rowStride, int rowOffset, int capacity, int lastN, float repeat, float presence, float frequency) =>
        Check(ns_f32_penalize_rows(_device, P(logits), P(work), P(history), P(length), rows, vocabulary, rowStride, rowOffset, capacity, lastN, repeat, presence,
            frequency), nameof(ns_f32_penalize_rows));

    public override void HistoryPush(Storage ids, Storage history, Storage length, int rows, int capacity) =>
        Check(ns_f32_history_push(_device, P(ids), P(history), P(length), rows, capacity), nameof(ns_f32_history_push));

    // ------------------------------------------------------------------------------------------------ graphs

    public override bool SupportsGraphs => true;

    public override void BeginCapture()
    {
        lock (_pool)
        {
            if (_captureFree is not null)
            {
                throw new InvalidOperationException("A graph is already being recorded on this device.");
            }

            _captureFree = [];
        }

        int result = ns_capture_begin(_device);
        if (result != 0)
        {
            lock (_pool)
            {
                _captureFree = null;
            }

            Check(result, nameof(ns_capture_begin));
        }
    }

    // The library hands back ONE handle for a recorded graph (it keeps the graph and its executable together): it
    // travels in the Executable slot, the Graph slot stays empty.
    public override (IntPtr Executable, IntPtr Graph, List<Storage> Owned) EndCapture()
    {
        var owned = TakeCaptureBlocks();
        int result = ns_capture_end(_device, out nint graph);
        if (result != 0)
        {
            owned.ForEach(o => o.Release());
            Check(result, nameof(ns_capture_end));
        }

        return (graph, IntPtr.Zero, owned);
    }

    public override List<Storage> AbortCapture()
    {
        var owned = TakeCaptureBlocks();
        ns_capture_abort(_device);
        return owned;
    }

    private List<Storage> TakeCaptureBlocks()
    {
        lock (_pool)
        {
            var owned = new List<Storage>();
            foreach (var (length, bucket) in _captureFree ?? [])
            {
                foreach (ulong pointer in bucket)
                {
                    // counted as in use again; releasing the storage later puts the block into the shared pool
                    _cached -= Bytes(length);
                    _inUse += Bytes(length);
                    owned.Add(new NsB200Storage(this, pointer, length));
                }
            }

            _captureFree = null;
            return owned;
        }
    }

    public override void ReplayGraph(IntPtr executable) => Check(ns_graph_launch(_device, executable), nameof(ns_graph_launch));

    public override void DestroyGraph(IntPtr executable, IntPtr graph)
    {
        if (executable != IntPtr.Zero)
        {
            ns_graph_destroy(executable);
        }
    }

    // ------------------------------------------------------------------------------------------------ outside the inference path

    public override void Unary(UnaryOp op, Storage x, Storage y, int n) => throw OffPath(nameof(Unary));

    public override void UnaryBackward(UnaryOp op, Storage x, Storage y, Storage dy, Storage dx, int n) => throw OffPath(nameof(UnaryBackward));

    public override void Axpy(Storage x, Storage y, int n, float alpha) => throw OffPath(nameof(Axpy));

    public override void MulAdd(Storage a, Storage b, Storage c, int n) => throw OffPath(nameof(MulAdd));

    public override void SumRows(Storage x, Storage y, int rows, int cols) => throw OffPath(nameof(SumRows));

    public override void Sum(Storage x, Storage result, int n, float scale) => throw OffPath(nameof(Sum));

    public override void AxpyAt(Storage x, Storage y, int offset, float alpha) => throw OffPath(nameof(AxpyAt));

    public override void SoftmaxBackward(Storage y, Storage dy, Storage dx, int rows, int cols, bool log) => throw OffPath(nameof(SoftmaxBackward));

    public override void ClassMatch(Storage predictions, Storage targets, Storage y, int rows, int cols, float threshold) => throw OffPath(nameof(ClassMatch));

    public override void NormStats(Storage x, Storage mean, Storage variance, Storage invStd, int outer, int groups, int inner, float eps) =>
        throw OffPath(nameof(NormStats));

    public override void NormApply(Storage x, Storage mean, Storage invStd, Storage y, int outer, int groups, int inner) => throw OffPath(nameof(NormApply));

    public override void NormBackward(Storage dxhat, Storage xhat, Storage sum1, Storage sum2, Storage invStd, Storage dx, int outer, int groups, int inner) =>
        throw OffPath(nameof(NormBackward));

    public override void GroupScaleShift(Storage x, Storage? scale, Storage? shift, Storage y, int n, int groups, int inner, bool accumulate) =>
        throw OffPath(nameof(GroupScaleShift));

    public override void GroupReduce(Storage a, Storage? b, Storage sumA, Storage? sumAB, int outer, int groups, int inner) => throw OffPath(nameof(GroupReduce));

    public override void InvSqrt(Storage x, Storage y, int n, float eps) => throw OffPath(nameof(InvSqrt));

    public override void ScatterAdd(Storage dy, Storage indices, Storage dtable, int count, int dim, int vocabulary) => throw OffPath(nameof(ScatterAdd));

    public override void Im2Col(Storage x, Storage cols, in ConvGeometry g) => throw OffPath(nameof(Im2Col));

    public override void Col2Im(Storage dcols, Storage dx, in ConvGeometry g) => throw OffPath(nameof(Col2Im));

    public override void MaxPool(Storage x, Storage y, Storage argmax, in ConvGeometry g) => throw OffPath(nameof(MaxPool));

    public override void MaxPoolBackward(Storage dy, Storage argmax, Storage dx, int count) => throw OffPath(nameof(MaxPoolBackward));

    public override void SumAxis(Storage x, Storage y, int outer, int dim, int inner, float scale, bool accumulate) => throw OffPath(nameof(SumAxis));

    public override void BroadcastAxis(Storage dy, Storage dx, int outer, int dim, int inner, float scale) => throw OffPath(nameof(BroadcastAxis));

    public override void SgdStep(Storage p, Storage g, Storage? v, int n, float lr, float momentum) => throw OffPath(nameof(SgdStep));

    public override void AdamStep(Storage p, Storage g, Storage m, Storage v, int n, float lr, float beta1, float beta2, float eps) => throw OffPath(nameof(AdamStep));

    public override void Dropout(Storage x, Storage y, int n, float p, uint seed) => throw OffPath(nameof(Dropout));

    public override void DropoutBackward(Storage dy, Storage dx, int n, float p, uint seed) => throw OffPath(nameof(DropoutBackward));
}
