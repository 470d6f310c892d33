/* Stand-in for the nanoarrow C library (see include/nanoarrow/nanoarrow.h). */
#include "nanoarrow/nanoarrow.h"

#include <errno.h>
#include <stdio.h>
#include <string.h>

ArrowErrorCode ArrowSchemaViewInit(struct ArrowSchemaView* view, const struct ArrowSchema* schema,
                                   struct ArrowError* error) {
  if (error != NULL) error->message[0] = '\0';
  if (schema == NULL || schema->release == NULL || schema->format == NULL) {
    if (error != NULL) snprintf(error->message, sizeof(error->message), "schema is released or has no format");
    return EINVAL;
  }
  view->schema = schema;
  const char* f = schema->format;
  enum ArrowType t = NANOARROW_TYPE_OTHER;
  if (f[0] != '\0' && f[1] == '\0') {
    switch (f[0]) {
      case 'n': t = NANOARROW_TYPE_NA; break;
      case 'b': t = NANOARROW_TYPE_BOOL; break;
      case 'c': t = NANOARROW_TYPE_INT8; break;
      case 'C': t = NANOARROW_TYPE_UINT8; break;
      case 's': t = NANOARROW_TYPE_INT16; break;
      case 'S': t = NANOARROW_TYPE_UINT16; break;
      case 'i': t = NANOARROW_TYPE_INT32; break;
      case 'I': t = NANOARROW_TYPE_UINT32; break;
      case 'l': t = NANOARROW_TYPE_INT64; break;
      case 'L': t = NANOARROW_TYPE_UINT64; break;
      case 'e': t = NANOARROW_TYPE_HALF_FLOAT; break;
      case 'f': t = NANOARROW_TYPE_FLOAT; break;
      case 'g': t = NANOARROW_TYPE_DOUBLE; break;
      case 'u': t = NANOARROW_TYPE_STRING; break;
      case 'z': t = NANOARROW_TYPE_BINARY; break;
      default: break;
    }
  } else if (strcmp(f, "+s") == 0) {
    t = NANOARROW_TYPE_STRUCT;
  }
  view->type = t;
  return NANOARROW_OK;
}

const char* ArrowErrorMessage(struct ArrowError* error) {
  return error == NULL ? "" : error->message;
}

const char* ArrowTypeString(enum ArrowType type) {
  switch (type) {
    case NANOARROW_TYPE_NA: return "na";
    case NANOARROW_TYPE_BOOL: return "bool";
    case NANOARROW_TYPE_UINT8: return "uint8";
    case NANOARROW_TYPE_INT8: return "int8";
    case NANOARROW_TYPE_UINT16: return "uint16";
    case NANOARROW_TYPE_INT16: return "int16";
    case NANOARROW_TYPE_UINT32: return "uint32";
    case NANOARROW_TYPE_INT32: return "int32";
    case NANOARROW_TYPE_UINT64: return "uint64";
    case NANOARROW_TYPE_INT64: return "int64";
    case NANOARROW_TYPE_HALF_FLOAT: return "half_float";
    case NANOARROW_TYPE_FLOAT: return "float";
    case NANOARROW_TYPE_DOUBLE: return "double";
    case NANOARROW_TYPE_STRING: return "string";
    case NANOARROW_TYPE_BINARY: return "binary";
    case NANOARROW_TYPE_STRUCT: return "struct";
    default: return "other";
  }
}
