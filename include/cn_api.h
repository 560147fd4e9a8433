/*
 * cn_api.h -- stand-in for the vendor driver header that the reference's
 * mlu_op.h includes (reference mlu_op.h:43).  A device is a CUDA device
 * ordinal.
 */
#ifndef MLUOP_B200_CN_API_H_
#define MLUOP_B200_CN_API_H_

typedef int CNdev;

#endif /* MLUOP_B200_CN_API_H_ */
