// Thin Swift host over libtmcuda's C ABI.
//
// Keeps the call shapes of the reference's Swift API for the hot path -
// `MetalCompiler.emit`, `MetalRuntime.makeLibrary/loadKernel/makeBuffer/launch`
// (Sources/TritonMetalCore/Runtime.swift:40-243, Compiler.swift:79-101 in the
// reference) - so tmbench and the test harness compile against it unchanged, while
// every call is one tm_* entry point.  Written for a Linux Swift toolchain; this
// repository's build image has none, so the file is not compiled here.
import CTMCuda
import Foundation

public enum CoreError: Error, CustomStringConvertible {
    case core(String)
    public var description: String {
        switch self { case .core(let message): return message }
    }
}

@inline(__always) private func takeString(_ pointer: UnsafeMutablePointer<CChar>?) -> String? {
    guard let pointer else { return nil }
    defer { tm_free(pointer) }
    return String(cString: pointer)
}

private func lastError() -> CoreError {
    .core(takeString(tm_last_error()) ?? "unknown error")
}

/// A device buffer both the host and the GPU address (`tm_alloc_buffer`).
public final class DeviceBuffer {
    public let handle: Int64
    public let length: Int
    init(handle: Int64, length: Int) { self.handle = handle; self.length = length }
    public func contents() -> UnsafeMutableRawPointer { tm_buffer_contents(handle)! }
    public func write(_ bytes: UnsafeRawBufferPointer, offset: Int = 0) throws {
        guard tm_buffer_write(handle, Int64(offset), bytes.baseAddress, Int64(bytes.count)) == 0
        else { throw lastError() }
    }
    public func read(into bytes: UnsafeMutableRawBufferPointer, offset: Int = 0) throws {
        guard tm_buffer_read(handle, Int64(offset), bytes.baseAddress, Int64(bytes.count)) == 0
        else { throw lastError() }
    }
    deinit { _ = tm_free_buffer(handle) }
}

public final class KernelLibrary {
    public let handle: Int64
    init(handle: Int64) { self.handle = handle }
    deinit { _ = tm_release_library(handle) }
}

public final class Pipeline {
    public let handle: Int64
    init(handle: Int64) { self.handle = handle }
    public var maxTotalThreadsPerThreadgroup: Int { Int(tm_kernel_max_threads(handle)) }
    /// Additive: causal masking for the attention kernels.
    public func setCausal(_ causal: Bool) throws {
        guard tmx_kernel_set_option(handle, "causal", causal ? 1 : 0) == 0 else { throw lastError() }
    }
    deinit { _ = tm_release_kernel(handle) }
}

public enum MetalCompiler {
    /// Triton IR text -> kernel descriptor text (the reference returns MSL here).
    public static func emitMSL(ttir: String, numSimdgroups: Int = 4) throws -> String {
        guard let text = takeString(ttir.withCString { tm_emit_msl($0, Int32(numSimdgroups)) })
        else { throw lastError() }
        return text
    }
    public static func kernelInfoJSON(ttir: String, numSimdgroups: Int = 4) throws -> String {
        guard let text = takeString(ttir.withCString { tm_kernel_info($0, Int32(numSimdgroups)) })
        else { throw lastError() }
        return text
    }
    public static func compileMSL(_ source: String) throws -> KernelLibrary {
        let handle = source.withCString { tm_compile_msl($0) }
        guard handle != 0 else { throw lastError() }
        return KernelLibrary(handle: handle)
    }
}

public enum MetalRuntime {
    public enum LaunchArgument {
        case buffer(DeviceBuffer)
        case int32(Int32)
        case int64(Int64)
        case float32(Float)
    }

    public static func defaultDeviceName() -> String? { takeString(tm_device_name()) }
    public static var unusableReason: String? { takeString(tm_unusable_reason()) }
    public static var isUsable: Bool { tm_is_usable() == 1 }

    public static func loadKernel(library: KernelLibrary, kernelName: String) throws -> Pipeline {
        let handle = kernelName.withCString { tm_load_kernel(library.handle, $0) }
        guard handle != 0 else { throw lastError() }
        return Pipeline(handle: handle)
    }

    public static func makeBuffer(length: Int) throws -> DeviceBuffer {
        let handle = tm_alloc_buffer(Int64(length))
        guard handle != 0 else { throw lastError() }
        return DeviceBuffer(handle: handle, length: length)
    }

    /// One dispatch, blocking until the GPU is done (tm_launch).  `threadgroups` keeps the
    /// reference's meaning: one program per BLOCK tile; y is batch*heads for attention.
    public static func launch(
        pipeline: Pipeline, threadgroups: (Int, Int, Int), threadsPerThreadgroup: Int,
        arguments: [LaunchArgument]
    ) throws {
        var kinds: [Int32] = []
        var values: [Int64] = []
        for argument in arguments {
            switch argument {
            case .buffer(let buffer): kinds.append(0); values.append(buffer.handle)
            case .int32(let v): kinds.append(1); values.append(Int64(v))
            case .float32(let v): kinds.append(2); values.append(Int64(v.bitPattern))
            case .int64(let v): kinds.append(3); values.append(v)
            }
        }
        let status = tm_launch(
            pipeline.handle, Int64(threadgroups.0), Int64(threadgroups.1), Int64(threadgroups.2),
            Int64(threadsPerThreadgroup), kinds, values, Int32(kinds.count))
        guard status == 0 else { throw lastError() }
    }
}
