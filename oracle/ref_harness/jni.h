/* Minimal stand-in for the JDK's <jni.h>, test infrastructure only.
 *
 * The reference's CUDA kernel file is written to be included from a JNI translation unit; one helper
 * in it takes a JNIEnv*.  No JDK exists on the build machine, so this header declares just enough of
 * the JNI vocabulary (scalar typedefs, opaque object handles, the JNIEnv members the included
 * reference headers name) for that file to compile.  Nothing here is ever called: the harness hands
 * device pointers straight to the reference's kernels and launch helpers.  The member functions are
 * declared and never defined on purpose.
 */
#pragma once
#include <stdint.h>

typedef int32_t jint;
typedef int64_t jlong;
typedef int8_t jbyte;
typedef uint8_t jboolean;
typedef uint16_t jchar;
typedef int16_t jshort;
typedef float jfloat;
typedef double jdouble;
typedef jint jsize;

class _jobject {};
typedef _jobject* jobject;
typedef jobject jclass;
typedef jobject jstring;
typedef jobject jarray;
typedef jarray jfloatArray;
typedef jarray jintArray;
typedef jarray jlongArray;
typedef jarray jbyteArray;
typedef jarray jdoubleArray;
typedef jarray jshortArray;
typedef jarray jbooleanArray;
typedef jarray jobjectArray;
typedef jobject jthrowable;

#define JNI_FALSE 0
#define JNI_TRUE 1
#define JNI_OK 0
#define JNI_COMMIT 1
#define JNI_ABORT 2
#define JNIEXPORT __attribute__((visibility("default")))
#define JNICALL
#define JNI_VERSION_1_8 0x00010008

struct JNIEnv {
    jfloat* GetFloatArrayElements(jfloatArray, jboolean*);
    void ReleaseFloatArrayElements(jfloatArray, jfloat*, jint);
    jint* GetIntArrayElements(jintArray, jboolean*);
    void ReleaseIntArrayElements(jintArray, jint*, jint);
    jlong* GetLongArrayElements(jlongArray, jboolean*);
    void ReleaseLongArrayElements(jlongArray, jlong*, jint);
    jbyte* GetByteArrayElements(jbyteArray, jboolean*);
    void ReleaseByteArrayElements(jbyteArray, jbyte*, jint);
    jshort* GetShortArrayElements(jshortArray, jboolean*);
    void ReleaseShortArrayElements(jshortArray, jshort*, jint);
    jdouble* GetDoubleArrayElements(jdoubleArray, jboolean*);
    void ReleaseDoubleArrayElements(jdoubleArray, jdouble*, jint);
    void* GetPrimitiveArrayCritical(jarray, jboolean*);
    void ReleasePrimitiveArrayCritical(jarray, void*, jint);
    jsize GetArrayLength(jarray);
    void* GetDirectBufferAddress(jobject);
    jlong GetDirectBufferCapacity(jobject);
    jclass FindClass(const char*);
    jint ThrowNew(jclass, const char*);
    jboolean ExceptionCheck();
    void DeleteLocalRef(jobject);
    jobject GetObjectArrayElement(jobjectArray, jsize);
    void GetFloatArrayRegion(jfloatArray, jsize, jsize, jfloat*);
    void SetFloatArrayRegion(jfloatArray, jsize, jsize, const jfloat*);
    void GetIntArrayRegion(jintArray, jsize, jsize, jint*);
    void SetIntArrayRegion(jintArray, jsize, jsize, const jint*);
};
struct JavaVM;
