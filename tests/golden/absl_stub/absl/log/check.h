// See status.h in this folder.
#pragma once
#include "absl/log/log.h"

#define CHECK(cond) \
  (cond) ? (void)0 : ::absl_stub::Voidify() & ::absl_stub::LogLine(true) << "check failed: " #cond " "
#define CHECK_OP_STUB(a, b, op) CHECK((a)op(b))
#define CHECK_EQ(a, b) CHECK_OP_STUB(a, b, ==)
#define CHECK_NE(a, b) CHECK_OP_STUB(a, b, !=)
#define CHECK_LT(a, b) CHECK_OP_STUB(a, b, <)
#define CHECK_LE(a, b) CHECK_OP_STUB(a, b, <=)
#define CHECK_GT(a, b) CHECK_OP_STUB(a, b, >)
#define CHECK_GE(a, b) CHECK_OP_STUB(a, b, >=)
#define DCHECK(cond) CHECK(cond)
#define DCHECK_EQ(a, b) CHECK_EQ(a, b)
#define DCHECK_LT(a, b) CHECK_LT(a, b)
#define DCHECK_LE(a, b) CHECK_LE(a, b)
#define DCHECK_GE(a, b) CHECK_GE(a, b)
#define DCHECK_GT(a, b) CHECK_GT(a, b)
#define DCHECK_NE(a, b) CHECK_NE(a, b)
