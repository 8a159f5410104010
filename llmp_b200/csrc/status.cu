// Status reporting and device probing shared by every entry point.
#include "common.cuh"

namespace llmp_b200 {

char* ErrorBuffer() {
  static thread_local char buffer[512] = "";
  return buffer;
}

int Reject(const char* format, ...) {
  va_list args;
  va_start(args, format);
  vsnprintf(ErrorBuffer(), 512, format, args);
  va_end(args);
  return LLMP_B200_REJECTED;
}

int Failed(cudaError_t error, const char* what) {
  snprintf(ErrorBuffer(), 512, "%s: %s (%s)", what, cudaGetErrorName(error),
           cudaGetErrorString(error));
  const int code = static_cast<int>(error);
  return code > 0 ? -code : -1;
}

namespace {
struct DeviceFacts {
  bool probed = false;
  int device = -1;
  int major = 0;
  int minor = 0;
  int sms = 0;
};
// Per host thread, per current device: the probe is two attribute reads.
DeviceFacts& Facts() {
  static thread_local DeviceFacts facts;
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess) {
    cudaGetLastError();
    facts = DeviceFacts{};
    facts.probed = true;
    return facts;
  }
  if (!facts.probed || facts.device != device) {
    facts = DeviceFacts{};
    facts.probed = true;
    facts.device = device;
    cudaDeviceGetAttribute(&facts.major, cudaDevAttrComputeCapabilityMajor, device);
    cudaDeviceGetAttribute(&facts.minor, cudaDevAttrComputeCapabilityMinor, device);
    cudaDeviceGetAttribute(&facts.sms, cudaDevAttrMultiProcessorCount, device);
    if (cudaGetLastError() != cudaSuccess) {
      facts.major = 0;
    }
  }
  return facts;
}
}  // namespace

int DeviceStatus() {
  const DeviceFacts& f = Facts();
  if (f.device < 0 || f.major != 10 || f.minor != 0) {
    snprintf(ErrorBuffer(), 512,
             "no compute-capability 10.0 device is current (device %d is %d.%d): this library "
             "has sm_100a code only and no fallback",
             f.device, f.major, f.minor);
    return LLMP_B200_NO_DEVICE;
  }
  return 0;
}

int SmCount() { return DeviceStatus() == 0 ? Facts().sms : 0; }

// Raised by a kernel whose bounded wait ran out; never by a healthy run.
__device__ unsigned int g_wait_timeouts = 0;

int ReadFaultCounter();

unsigned int* FaultCounter() {
  static thread_local int cached_device = -1;
  static thread_local unsigned int* cached = nullptr;
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess) return nullptr;
  if (device != cached_device) {
    void* address = nullptr;
    if (cudaGetSymbolAddress(&address, g_wait_timeouts) != cudaSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    cached = static_cast<unsigned int*>(address);
    cached_device = device;
  }
  return cached;
}

int ClearFaultCounter() {
  const int before = ReadFaultCounter();
  const unsigned int zero = 0;
  if (before < 0 || cudaMemcpyToSymbol(g_wait_timeouts, &zero, sizeof(zero)) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  return before;
}

int ReadFaultCounter() {
  unsigned int count = 0;
  if (cudaMemcpyFromSymbol(&count, g_wait_timeouts, sizeof(count)) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  return static_cast<int>(count);
}

}  // namespace llmp_b200

extern "C" {
int llmp_b200_available(void) { return llmp_b200::DeviceStatus() == 0 ? 1 : 0; }
int llmp_b200_sm_count(void) { return llmp_b200::SmCount(); }
const char* llmp_b200_last_error(void) { return llmp_b200::ErrorBuffer(); }
int llmp_b200_device_faults(void) {
  return llmp_b200::DeviceStatus() != 0 ? 0 : llmp_b200::ReadFaultCounter();
}
int llmp_b200_device_faults_clear(void) {
  return llmp_b200::DeviceStatus() != 0 ? 0 : llmp_b200::ClearFaultCounter();
}
}
