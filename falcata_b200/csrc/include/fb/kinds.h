// Small integer codes shared by the host code, the device kernels and the Python layer.
#pragma once

namespace fb {

enum ObjKind : int {
  kObjL2 = 0, kObjL1 = 1, kObjHuber = 2, kObjFair = 3, kObjPoisson = 4, kObjQuantile = 5, kObjMape = 6,
  kObjGamma = 7, kObjTweedie = 8, kObjBinary = 9, kObjMulticlass = 10, kObjMulticlassOVA = 11, kObjXent = 12,
  kObjXentLambda = 13, kObjLambdarank = 14, kObjXendcg = 15, kObjCustom = 16, kObjMultiReg = 17
};

enum MetricKind : int {
  kMetL2 = 0, kMetRMSE = 1, kMetL1 = 2, kMetBinaryLogloss = 3, kMetBinaryError = 4, kMetAUC = 5,
  kMetMultiLogloss = 6, kMetMultiError = 7, kMetNDCG = 8
};

// Status codes written by device kernels into the status word (0 = ok). A kernel that gives up on
// a bounded wait records where and returns; it never traps.
enum DeviceStatus : int {
  kStatusOk = 0,
  kStatusWaitTimeout = 1,     // a cross-rank flag did not arrive within the spin budget
  kStatusBoundsViolation = 2, // a checked index was out of range (debug builds)
  kStatusOverflow = 3,        // a level needed more descriptors than were allocated
};

}  // namespace fb
